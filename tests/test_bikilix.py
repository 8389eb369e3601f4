"""The Bikilix decoder against its plain implementation (``plain_bikilix``): each mechanism alone (the norm pair around
a sub-layer, the merge of the stream with its origin, neighbouring columns rotated, frequencies stretched by index,
windowed attention, gated latent attention, the per-head value product, the relu^2 feed-forward, the router's corrected
choice among groups, the clamped experts), then whole models through trace replay (whole, decoded one by one, in
portions down to two tokens, mixed batches on a pool that runs full, long prompts on the tensor-core kernels, randomly
drawn configurations) and greedy generation through the engine and the command line.

Configurations and weights are made here.  Score factors are large enough that much of a query's weight sits on a few
keys; where random weights would still hide a fault (a key just outside a window, a key hundreds of tokens back, a group
of experts that must stay closed) the test makes rows or weights so that it shows."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_bikilix as plain
from plain_qwen3 import read_model_folder
from tiny_configs import random_tokens

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = [torch.float32, torch.bfloat16]


def rot(base, dims, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling:
        out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return out


def attn(heads, kv_heads, dim, vdim, scale, rotation, window):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rotation}
    if window:
        mixer["mask"] = {"size": window}
    return {"type": "attention", "mixer": mixer}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base=10000.0, scaling=None):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank,
                                                  "kv_rank": kv_rank, "scale": scale, "rot": rot(base, rot_dim, scaling)}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, limit, experts, top, count, keep):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}


def layer(entry, mlp):
    return {**entry, "mlp": mlp}


# A: sizes in multiples of 8; the looped stretch in the middle, a layer ahead of it and one behind; a window of two and
# a half pages; a latent layer without feed-forward; experts in 4 groups of which 2 stay open.  B: nothing a multiple
# of 8, the whole model looped three times, one kv head for six query heads, a window shorter than a page, values wider
# than keys, one group of experts (no limit on the choice) and a layer whose tokens use ONE expert of two groups of which
# both stay open, stretched frequencies that reach the clamp on both sides.
CONFIG_A = {
    "architecture": "Bikilix", "width": 64, "vocab": 200, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.5},
    "layers": [
        layer(attn(4, 2, 16, 8, 3.0, rot(500.0, 8), 10), dense(96)),
        layer(latent(4, 8, 8, 16, 24, 16, 1.5, base=300.0, scaling=(4.0, 32, 8.0, 1.0)), moe(16, 0.4, 8, 2, 4, 2)),
        layer(latent(2, 16, 4, 8, 16, 24, 1.2), None),
        layer(attn(2, 2, 32, 32, 2.0, rot(10000.0, 32), 33), moe(24, 1.0, 6, 3, 3, 2)),
    ],
    "loop": {"start": 1, "stop": 3, "times": 2},
}
CONFIG_B = {
    "architecture": "Bikilix", "width": 100, "vocab": 131, "norm": {"eps": 1e-3}, "embedding": {"scale": 0.7},
    "layers": [
        layer(latent(6, 10, 6, 12, 20, 18, 1.2, base=50.0, scaling=(2.0, 16, 4.0, 0.5)), moe(12, 0.25, 5, 2, 1, 1)),
        layer(attn(6, 1, 12, 20, 2.0, rot(77.0, 4), 5), moe(20, 2.0, 6, 1, 2, 2)),
        layer(attn(3, 3, 10, 10, 2.5, rot(50.0, 10), 64), dense(52)),
    ],
    "loop": {"start": 0, "stop": 3, "times": 3},
}
TINY = {"A": (CONFIG_A, 4, 11), "B": (CONFIG_B, 8, 12)}  # name -> (config, page size, seed)


def write_model(folder, raw, seed, std=0.08):
    """Random weights; the norms' stored tensors (the weights minus one) and the routers' corrections are made larger
    than the random-weights mode makes them, so that a lost ``1 +`` or a lost correction shows and the experts' choice
    scores lie far enough apart that few choices are close calls."""
    import kirai_b200  # noqa: F401
    from kirai_b200.registry import config_from_dict, plan_for_config
    from kirai_b200.weights.random_init import random_tensors
    from kirai_b200.weights.safetensors_io import write_safetensors

    cfg = config_from_dict(raw)
    tensors = random_tensors(plan_for_config(cfg).weight_specs(), seed, std=std, norm_jitter=0.3, dtype=torch.bfloat16)
    for name in tensors:
        if ".norm" in name and not name.endswith((".dq.norm", ".dkv.norm")) or name == "loop.step":
            tensors[name] = (tensors[name].float() * 4).to(torch.bfloat16)
        if name.endswith(".correction"):
            tensors[name] = (tensors[name].float() * 8 * 0.08 / std).to(torch.bfloat16)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(cfg.to_dict(), handle, indent=2)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors, metadata={"format": "pt"})


def tolerance(dtype, reference):
    dtype = {torch.float32: "float32", torch.bfloat16: "bfloat16"}.get(dtype, dtype)
    peak = float(np.abs(np.asarray(reference)).max())
    return 3e-5 * max(1.0, peak) if dtype == "float32" else 0.05 * peak


def close(dtype, got, expected, what, rows=None):
    got, expected = np.asarray(got, dtype=np.float64), np.asarray(expected, dtype=np.float64)
    assert got.shape == expected.shape, what
    diff = np.abs(got - expected)
    if rows is not None:
        diff = diff[np.asarray(rows)]
    worst = float(diff.max()) if diff.size else 0.0
    assert worst <= tolerance(dtype, expected), f"{what}: max abs diff {worst} (bound {tolerance(dtype, expected)})"


# --------------------------------------------------------------------------- no GPU
def test_config_reads_every_size_and_round_trips():
    import kirai_b200  # noqa: F401
    from kirai_b200.config.base import ConfigError
    from kirai_b200.parts.base import KVCacheNeed
    from kirai_b200.registry import config_from_dict, plan_for_config

    for raw in (CONFIG_A, CONFIG_B):
        cfg = config_from_dict(raw)
        assert cfg.to_dict() == raw and config_from_dict(cfg.to_dict()) == cfg
        assert [(n, list(i)) for n, i in cfg.passes()] == plain.passes(raw)
        plan = plan_for_config(cfg)
        runs = [index for _, indices in plain.passes(raw) for index in indices]
        assert [call.block for call in plan.order] == runs and len(plan.cache_needs) == len(runs)
        # a pass of the looped stretch enters through the merge with its own row of the step table
        firsts = [call.enter for call in plan.order if call.enter is not None]
        assert firsts == [(0, t) for t in range(raw["loop"]["times"])]
        assert all((call.enter is not None) == (call.block == raw["loop"]["start"]) for call in plan.order)
        for call in plan.order:
            m, need = raw["layers"][call.block]["mixer"], plan.cache_needs[call.cache]
            if raw["layers"][call.block]["type"] == "latent_attention":
                assert isinstance(need, KVCacheNeed) and need.kv_heads == 1 and need.key_dim == m["kv_rank"] + m["rot_dim"] and need.window is None
            else:
                assert isinstance(need, KVCacheNeed) and need.kv_heads == m["kv_heads"] and need.window == m["mask"]["size"]
        names = set(plan.weight_specs())
        assert {"embed", "loop.in", "loop.step", "final.norm"} <= names and "head" not in names
        for i, entry in enumerate(raw["layers"]):
            has = entry["mlp"] is not None
            assert {f"l{i}.norm1", f"l{i}.norm1b"} <= names and (f"l{i}.norm2" in names) == has == (f"l{i}.norm2b" in names)
            assert (f"l{i}.mlp.up" in names) == (has and entry["mlp"]["kind"] == "dense")
            assert (f"l{i}.mlp.correction" in names) == (has and entry["mlp"]["kind"] == "moe") == (f"l{i}.mlp.e0.gate" in names)
            assert (f"l{i}.mix.q.b" in names) == (entry["type"] == "attention") and (f"l{i}.mix.g" in names) == (entry["type"] != "attention")
    no_loop = json.loads(json.dumps(CONFIG_A))
    del no_loop["loop"]
    plan = plan_for_config(config_from_dict(no_loop))
    assert not plan.entries and "loop.in" not in plan.weight_specs() and [c.block for c in plan.order] == [0, 1, 2, 3]
    for change in (lambda r: r["layers"][0].update(type="mingru"),
                   lambda r: r["layers"][0]["mixer"]["rot"].update(dims=7),
                   lambda r: r["layers"][0]["mixer"].update(kv_heads=3),
                   lambda r: r["layers"][1]["mixer"].update(rot_dim=4),
                   lambda r: r.update(loop={"start": 2, "stop": 9, "times": 2}),
                   lambda r: r["layers"][0]["mlp"].update(kind="gated"),
                   lambda r: r["layers"][1]["mlp"]["router"]["groups"].update(count=3),
                   lambda r: r["layers"][1]["mlp"]["router"].update(top=5),
                   lambda r: r["layers"][1]["mlp"]["expert"].update(limit=0.0)):
        bad = json.loads(json.dumps(CONFIG_A))
        change(bad)
        with pytest.raises(ConfigError):
            config_from_dict(bad)


def test_frequencies_stretched_by_index_and_the_order_of_neighbours():
    import kirai_b200  # noqa: F401
    from kirai_b200.parts import RotaryEmbedding

    for dims, base, scaling in ((8, 300.0, (4.0, 32, 8.0, 1.0)), (6, 50.0, (2.0, 16, 4.0, 0.5)), (32, 250000.0, (6.0, 1024, 16.0, 2.0)),
                                (16, 10000.0, None)):
        table, amplitude = plain.pair_frequencies(rot(base, dims, scaling))
        part = RotaryEmbedding(dims, base, dims, scaling=dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None,
                               precise=True, pairing="neighbours")
        assert torch.equal(part.frequencies(), table.to(torch.float32)) and abs(part.amplitude - amplitude) < 1e-12
    # the first table: the fastest pair keeps its frequency, the slowest is divided by the factor, one lies between
    table, amplitude = plain.pair_frequencies(rot(300.0, 8, (4.0, 32, 8.0, 1.0)))
    raw = [300.0 ** (-2.0 * i / 8) for i in range(4)]
    assert table[0] == raw[0] and abs(float(table[3]) - raw[3] / 4) < 1e-15 and raw[1] / 4 < float(table[1]) < raw[1]
    assert abs(amplitude - (0.1 * math.log(4.0) + 1)) < 1e-15
    # rotating halves of rows put in head_order equals rotating neighbours, put in the same order afterwards
    part = RotaryEmbedding(12, 77.0, 8, pairing="neighbours")
    order = part.head_order()
    assert order.tolist() == [0, 2, 4, 6, 1, 3, 5, 7, 8, 9, 10, 11]
    assert part.row_order(2).tolist() == order.tolist() + [12 + c for c in order.tolist()]
    x = torch.randn((5, 1, 12), generator=torch.Generator().manual_seed(0), dtype=torch.float64)
    positions = torch.tensor([0, 1, 7, 300, 4096])
    want = plain.rotate_neighbours(x, positions, rot(77.0, 8))[..., order]
    y = x[..., order].clone()
    angle = (positions.to(torch.float32)[:, None] * part.frequencies()[None, :]).double()[:, None, :]
    u, v = y[..., :4].clone(), y[..., 4:8].clone()
    y[..., :4], y[..., 4:8] = u * angle.cos() - v * angle.sin(), v * angle.cos() + u * angle.sin()
    assert float((y - want).abs().max()) < 1e-12


def test_plain_router_keeps_closed_groups_closed_also_below_zero():
    """Six experts in three groups, one group open, two experts a token.  Corrections push every choice score below
    zero; the open group's two experts must be chosen although a closed group holds the largest single score, and
    a masked score that counted as 0 would win over all of them."""
    mlp = moe(4, 1.0, 6, 2, 3, 1)
    w = {"m.router": torch.zeros((6, 3), dtype=torch.float64), "m.correction": torch.tensor([-2.0, -2.1, -1.0, -5.0, -3.0, -3.0], dtype=torch.float64)}
    ids, weights = plain.router_choice(torch.ones((2, 3), dtype=torch.float64), w, mlp, "m.")
    # sums of the two largest: group 0 -3.1, group 1 -5, group 2 -5: group 0 is open although expert 2 stands highest
    assert ids.tolist() == [[0, 1], [0, 1]] and torch.allclose(weights, torch.full((2, 2), 0.5, dtype=torch.float64))


def test_plain_attention_is_peaky_reaches_back_and_feels_its_window(tmp_path):
    """What makes the comparisons below sharp: the heaviest key of many queries carries much of the weight; in the latent
    layers it often lies many pages back; and a window one token wider or narrower moves the logits by far more than
    any bound used below."""
    write_model(str(tmp_path), CONFIG_A, 11)
    raw, weights = read_model_folder(str(tmp_path))
    tokens = random_tokens(75, raw["vocab"], 200)
    w = {k: v.double() for k, v in weights.items()}
    n = plain.unit_norm(w["embed"][tokens] * 2.5, w["l1.norm1"], 1e-5, 1.0)
    probabilities = []
    plain.latent_attention(n, w, raw["layers"][1]["mixer"], "l1.mix.", 1e-5, probabilities)
    far = sum(int(((p.max(dim=1).values > 0.3) & (torch.arange(75) - p.argmax(dim=1) > 16)).sum()) for p in probabilities)
    assert far >= 5
    logits = plain.forward(raw, weights, tokens)
    for size in (9, 11):
        other = json.loads(json.dumps(raw))
        other["layers"][0]["mixer"]["mask"]["size"] = size
        assert float((plain.forward(other, weights, tokens) - logits).abs().max()) > 5 * tolerance("bfloat16", logits.numpy())


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [64, 100, 7, 4096 + 24])
def test_norm_on_an_output_then_the_next_norm_in_one_pass(dtype, width):
    """stream += normb(y), then norm(stream): as one kernel (what a sandwich block leaves is taken by the next norm), for
    chosen rows without touching the stream, and settled by itself; weights are stored as their distance from one."""
    from part_helpers import load_part
    from kirai_b200.parts import RMSNorm

    after, reader = RMSNorm("b", width, 1e-4, centre=1.0), RMSNorm("n", width, 1e-5, centre=1.0)
    wb = load_part(after, dtype, seed=width)["b"].double() * 10
    wn = load_part(reader, dtype, seed=width + 1)["n"].double() * 10
    after.weight, reader.weight = (wb.float() + 1).cuda(), (wn.float() + 1).cuda()
    g = torch.Generator().manual_seed(width)
    x = torch.randn((9, width), generator=g) * 3 + 1.5
    y = torch.randn((9, width), generator=g) * 20
    total = x.double() + plain.unit_norm(y.double(), wb, 1e-4, 1.0)
    resid = x.cuda()
    got = reader.add_forward(resid, after.normed_sum(y.cuda()))
    close(torch.float32, resid.cpu(), total, "the stream")
    close(dtype, got.float().cpu(), plain.unit_norm(total, wn, 1e-5, 1.0), "normed rows")
    rows = torch.tensor([7, 2, 2], dtype=torch.int32).cuda()
    before = resid.clone()
    picked = reader.add_forward_rows(resid, after.normed_sum(y.cuda()), rows)
    assert torch.equal(resid, before)
    twice = total + plain.unit_norm(y.double(), wb, 1e-4, 1.0)
    close(dtype, picked.float().cpu(), plain.unit_norm(twice, wn, 1e-5, 1.0)[[7, 2, 2]], "chosen rows")
    after.normed_sum(y.cuda()).settle(resid, reader.rt.ops)
    close(torch.float32, resid.cpu(), twice, "settled")
    # a stored zero is a weight of one
    after.weight = torch.ones(width).cuda()
    close(dtype, after.forward(x.cuda()).float().cpu(), plain.unit_norm(x.double(), torch.zeros(width, dtype=torch.float64), 1e-4, 1.0), "plain")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [64, 100, 24])
def test_stream_merges_with_its_origin(dtype, width):
    """x <- W [x; x0] + b_t for three passes over the same origin: after nothing, after a norm's output that is still to
    be added, and after plain rows that are still to be added."""
    from part_helpers import load_part
    from kirai_b200.parts import RMSNorm, StreamMerge

    merge, after = StreamMerge("in", width, "step", 3), RMSNorm("b", width, 1e-5, centre=1.0)
    w = {k: v.double() for k, v in load_part(merge, dtype, seed=width).items()}
    w["step"] = w["step"] * 20
    merge.bias = w["step"].float().cuda()
    wb = load_part(after, dtype, seed=1)["b"].double()
    g = torch.Generator().manual_seed(3)
    origin = (torch.randn((11, width), generator=g) * 2).to(dtype).float()
    y = torch.randn((11, width), generator=g) * 7
    delta = torch.randn((11, width), generator=g).to(dtype)

    def merged(x, t):
        return torch.cat([x, origin.double()], dim=1) @ w["in"].T + w["step"][t]

    pair = merge.begin(origin.cuda())
    resid, left = merge.forward(origin.cuda().clone(), None, pair, 0)
    assert left is None and resid.dtype == torch.float32
    expected = merged(origin.double(), 0)
    close(dtype, resid.cpu(), expected, "first pass")
    # the stream as the kernels hold it goes on; the comparison follows the plain numbers
    stream = resid.clone()
    resid, _ = merge.forward(stream, after.normed_sum(y.cuda()), pair, 1)
    expected = merged(expected + plain.unit_norm(y.double(), wb, 1e-5, 1.0), 1)
    close(dtype, resid.cpu(), expected, "second pass")
    resid, _ = merge.forward(resid, delta.cuda(), pair, 2)
    close(dtype, resid.cpu(), merged(expected + delta.double(), 2), "third pass")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,ff,tokens", [(64, 96, 13), (100, 52, 13), (24, 7, 5), (256, 384, 300)])
def test_relu_squared_feed_forward(dtype, width, ff, tokens):
    from part_helpers import load_part
    from kirai_b200.parts import PlainMLP

    part = PlainMLP("f.", width, ff, "relu2", names={"up": "up", "down": "down"}, out_dtype=torch.float32)
    w = {k: v.double() for k, v in load_part(part, dtype, seed=ff).items()}
    x = (torch.randn((tokens, width), generator=torch.Generator().manual_seed(ff)) * 6).to(dtype)
    got = part.forward(x.cuda(), None)
    assert got.dtype == torch.float32
    close(dtype, got.cpu(), plain.dense_ffn(x.double(), w, "f."), "feed-forward")


def _experts_part(mlp, width):
    import kirai_b200  # noqa: F401
    from kirai_b200.config.bikilix import BikilixConfig
    from kirai_b200.models.bikilix import feed_forward_for_layer

    raw = {"architecture": "Bikilix", "width": width, "vocab": 8, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
           "layers": [layer(attn(1, 1, 8, 8, 1.0, rot(100.0, 2), 4), mlp)]}
    cfg = BikilixConfig.from_dict(raw)
    return feed_forward_for_layer(cfg, cfg.layers[0], "m.")


EXPERT_CASES = [
    (moe(16, 0.4, 8, 2, 4, 2), 64, 40),
    (moe(12, 0.25, 5, 2, 1, 1), 100, 40),      # one group: no limit on the choice
    (moe(20, 2.0, 6, 1, 2, 2), 36, 40),        # every group open, one expert a token
    (moe(8, 1.3, 15, 3, 5, 2), 48, 1300),      # the many-token router kernel
    (moe(8, 0.7, 6, 4, 6, 5), 24, 9),          # groups of one expert
    (moe(128, 1.0, 8, 2, 4, 2), 128, 700),     # rows sorted by expert on the tensor cores (bfloat16)
    (moe(16, 0.6, 40, 4, 5, 3), 64, 200),      # more experts than a warp has lanes
]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mlp,width,tokens", EXPERT_CASES, ids=[f"experts{i}" for i in range(len(EXPERT_CASES))])
def test_experts_chosen_by_corrected_scores_among_groups(dtype, mlp, width, tokens):
    """The routed feed-forward alone.  Corrections as large as the scores' spread, so that choice and weights part; inputs
    large enough that gate and up values pass the limit on both sides.  In bfloat16, tokens whose choice is a close call
    are left out (their rounding may fall either way)."""
    from part_helpers import load_part

    part = _experts_part(mlp, width)
    w = {k: v.double() for k, v in load_part(part, dtype, seed=width).items()}
    w["m.correction"] = w["m.correction"] * 6
    part.correction = w["m.correction"].float().cuda()
    part.rule["correction"] = part.correction
    x = (torch.randn((tokens, width), generator=torch.Generator().manual_seed(tokens)) * 5).to(dtype)
    margins = []
    expected = plain.routed_ffn(x.double(), w, mlp, "m.", margins)
    ids, _ = plain.router_choice(x.double(), w, mlp, "m.")
    plain_scores = torch.sigmoid(x.double() @ w["m.router"].T)
    assert not torch.equal(ids.sort(dim=1).values, plain_scores.topk(mlp["router"]["top"], dim=1).indices.sort(dim=1).values)  # the correction matters
    gate = x.double() @ w["m.e0.gate"].T
    assert float(gate.max()) > mlp["expert"]["limit"] and float(gate.min()) < -mlp["expert"]["limit"]
    sure = (margins[0] > 0.02).numpy() if dtype == torch.bfloat16 else np.ones(tokens, bool)
    assert sure.mean() > 0.6
    got = part.forward(x.cuda(), None)
    assert got.dtype == torch.float32
    close(dtype, got.cpu(), expected, "all tokens at once", rows=sure)
    few = part.forward(x[:3].cuda(), None)
    close(dtype, few.cpu(), expected[:3], "three tokens", rows=sure[:3])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_router_leaves_closed_groups_closed_also_below_zero(dtype):
    """The hand-made case of the plain test through the kernels, in both router kernels and the choice alone."""
    from kirai_b200.csrc import ops

    correction = torch.tensor([-2.0, -2.1, -1.0, -5.0, -3.0, -3.0]).cuda()
    rule = {"correction": correction, "groups": 3, "keep": 1}
    for tokens in (2, 900):
        x = torch.ones((tokens, 8), dtype=dtype).cuda()
        gates, ids, weights = ops.router_gates(x, torch.zeros((6, 8)).cuda(), 2, True, rule=rule)
        assert ids.cpu().tolist() == [[0, 1]] * tokens and torch.equal(weights.cpu(), torch.full((tokens, 2), 0.5))
        assert torch.equal(gates.cpu(), torch.tensor([[0.5, 0.5, 0, 0, 0, 0]]).expand(tokens, 6))
    _, ids, weights = ops.router_choose_(torch.zeros((5, 6)).cuda(), 2, True, rule=rule)
    assert ids.cpu().tolist() == [[0, 1]] * 5 and torch.equal(weights.cpu(), torch.full((5, 2), 0.5))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,used,pad,n,tokens", [(4, 16, 24, 16, 7), (3, 18, 24, 12, 40), (2, 600, 608, 40, 19), (16, 96, 128, 32, 300), (1, 5, 8, 3, 1),
                                                     (16, 192, 256, 64, 700), (3, 18, 24, 12, 257)])
def test_a_product_per_head_with_its_gate(dtype, heads, used, pad, n, tokens):
    """On the CUDA cores, and (bfloat16, many tokens, given the matrices with zero columns up to the padded width) as a
    grouped product on the tensor cores with the heads as groups; columns beyond a head's used ones do not count."""
    from kirai_b200.csrc import ops

    g = torch.Generator().manual_seed(heads * n)
    x = torch.randn((tokens, heads, pad), generator=g).to(dtype)
    w = (torch.randn((heads, n, used), generator=g) / used ** 0.5).to(dtype)
    wide = torch.randn((tokens, heads * n + 5), generator=g) * 3
    expected = torch.einsum("thk,hnk->thn", x[..., :used].double(), w.double()).reshape(tokens, heads * n)
    got = ops.head_linear_gate(x.reshape(tokens, heads * pad).cuda(), w.cuda(), heads, used)
    close(dtype, got.float().cpu(), expected, "the product alone")
    gate = wide.cuda()[:, 5:]  # a run of columns of a wider product
    got = ops.head_linear_gate(x.reshape(tokens, heads * pad).cuda(), w.cuda(), heads, used, gate)
    close(dtype, got.float().cpu(), expected * torch.sigmoid(wide[:, 5:].double()), "with its gate")
    if dtype == torch.bfloat16:
        padded = torch.zeros((heads * n, pad), dtype=dtype)
        padded[:, :used] = w.reshape(heads * n, used)
        for g in (None, gate):
            got = ops.head_linear_gate(x.reshape(tokens, heads * pad).cuda(), w.cuda(), heads, used, g, padded_weight=padded.cuda())
            factor = 1.0 if g is None else torch.sigmoid(wide[:, 5:].double())
            close(dtype, got.float().cpu(), expected * factor, "given the padded matrices")
        if tokens >= ops.HEAD_GROUPED_MIN_ROWS and pad % 8 == 0:
            assert ops.launch_counts.get("kirai_head_major_bf16", 0) > 0


def _mixer_part(entry, width):
    import kirai_b200  # noqa: F401
    from kirai_b200.config.bikilix import BikilixConfig
    from kirai_b200.models.bikilix import mixer_for_layer

    raw = {"architecture": "Bikilix", "width": width, "vocab": 8, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
           "layers": [layer(entry, None)]}
    cfg = BikilixConfig.from_dict(raw)
    return mixer_for_layer(cfg, cfg.layers[0], "a."), raw["layers"][0]


def _plain_mixer(raw, x, w, probabilities=None):
    if raw["type"] == "attention":
        return plain.window_attention(x, w, raw["mixer"], "a.", probabilities)
    return plain.latent_attention(x, w, raw["mixer"], "a.", 1e-5, probabilities)


def _run_part(part, session, x, cuts, name="s"):
    """The part's output for rows x of one request, cut into steps of the given sizes."""
    out, start = [], 0
    for size in cuts:
        batch = session.batch([(name, size)])
        out.append(part.forward(x[start : start + size].cuda(), batch, session.cache.layer_view(0)).float().cpu())
        session.commit()
        start += size
    session.cache.close(session.requests.pop(name))
    return torch.cat(out)


PART_CASES = [
    (attn(4, 2, 16, 8, 3.0, rot(500.0, 8), 10), 64, 4),
    (attn(6, 1, 12, 20, 4.0, rot(77.0, 4), 5), 100, 8),
    (attn(2, 2, 32, 32, 2.0, rot(10000.0, 32), 33), 64, 4),
    (attn(3, 3, 10, 10, 2.5, rot(50.0, 10), 1), 24, 2),           # a window of one: every token sees itself alone
    (attn(8, 2, 64, 64, 0.8, rot(10000.0, 48), 48), 128, 16),
    (attn(6, 2, 128, 128, 0.5, rot(2e5, 64), 200), 96, 16),       # a window wider than the sequence
    (attn(4, 2, 256, 136, 0.4, rot(10000.0, 64), 40), 128, 16),
    (attn(2, 1, 24, 24, 1.0, rot(100.0, 8), None), 40, 4),        # no mask: every earlier token
    (latent(4, 8, 8, 16, 24, 16, 1.5, base=300.0, scaling=(4.0, 32, 8.0, 1.0)), 64, 4),
    (latent(6, 10, 6, 12, 20, 18, 1.2, base=50.0, scaling=(2.0, 16, 4.0, 0.5)), 100, 8),
    (latent(20, 16, 16, 8, 32, 48, 0.9), 64, 16),
    (latent(1, 24, 2, 24, 8, 30, 1.0), 40, 2),
    (latent(8, 32, 64, 32, 64, 192, 0.6, scaling=(8.0, 64, 32.0, 1.0)), 128, 16),   # a cached row of 256 columns
    (latent(4, 16, 32, 24, 40, 168, 0.6), 96, 8),                                   # a row of 200 columns
    (latent(2, 32, 16, 40, 32, 280, 0.5), 64, 16),                                  # a row beyond the tensor-core kernels
]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("entry,width,page", PART_CASES, ids=[f"{e['type']}{i}" for i, (e, _, _) in enumerate(PART_CASES)])
def test_attention_parts_whole_in_portions_and_one_by_one(dtype, entry, width, page):
    from part_helpers import Session, load_part

    part, raw = _mixer_part(entry, width)
    w = {k: v.double() for k, v in load_part(part, dtype, seed=width + page).items()}
    tokens = 90
    x = (torch.randn((tokens, width), generator=torch.Generator().manual_seed(page)) * 1.5).to(dtype)
    expected = _plain_mixer(raw, x.double(), w)
    session = Session([part.cache_need()], dtype, page_size=page, num_pages=2 * (-(-tokens // page)), num_slots=2)
    for cuts in ([tokens], [37, 2, 19, 1, 1, 3, 27], [80] + [1] * 10, [2] * 45):
        got = _run_part(part, session, x, cuts)
        assert part.out_dtype == torch.float32
        close(dtype, got, expected, f"cut as {cuts[:4]}...")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,page", [(48, 16), (21, 16), (16, 16), (5, 8)])
def test_keys_just_inside_and_just_outside_the_window_show(dtype, window, page):
    """Row 20 gets a component thirty times the size of a row that the key matrix cannot see (it lies in the matrix's
    null space) and the value matrix can: its key is an ordinary key, its value swamps whoever attends to it.  Every
    query head's matrix repeats the key matrix and the rows at the window's edge repeat row 20 as it was, so that
    their queries equal that key up to the few rotated columns and give it a third of their weight.  With a window of
    W, queries 20 .. 20 + W - 1 see row 20 and query 20 + W must not.  In a prompt portion that crosses the edge, in
    portions cut at the edge, and decoded one by one; the windows end inside a page, on a page's border and span
    several pages."""
    from part_helpers import Session, load_part
    from kirai_b200.weights.random_init import random_tensors

    part, raw = _mixer_part(attn(8, 1, 64, 64, 0.1, rot(10000.0, 8), window), 128)
    tensors = random_tensors(part.weight_specs(), 9, std=0.08, norm_jitter=0.1, dtype=torch.bfloat16)
    for head in range(8):
        tensors["a.q"][64 * head : 64 * head + 64] = tensors["a.k"]
        tensors["a.q.b"][64 * head : 64 * head + 64] = tensors["a.k.b"]
    w = {k: v.double() for k, v in load_part(part, dtype, seed=9, tensors=tensors).items()}
    edge = 20 + window
    x = torch.randn((90, 128), generator=torch.Generator().manual_seed(2)) * 1.5
    x[edge - 1] = x[20]
    x[edge] = x[20]
    unseen = torch.linalg.svd(w["a.k"]).Vh[-1]  # W_k [64, 128] times this direction is zero
    x[20] += (30 * 1.5 * 128 ** 0.5 * unseen).float()
    x = x.to(dtype)
    probabilities = []
    expected = plain.window_attention(x.double(), w, raw["mixer"], "a.", probabilities)
    assert float(probabilities[0][edge - 1, 20]) > 0.3
    off_by_one = json.loads(json.dumps(raw["mixer"]))
    for size in (window - 1, window + 1):
        off_by_one["mask"]["size"] = size
        wrong = plain.window_attention(x.double(), w, off_by_one, "a.")
        assert float((wrong - expected)[edge - 2 : edge + 2].abs().max()) > 3 * tolerance(dtype, expected.numpy())
    session = Session([part.cache_need()], dtype, page_size=page, num_pages=2 * (-(-90 // page)), num_slots=2)
    for cuts in ([90], [edge - 1, 2, 90 - edge - 1], [edge, 90 - edge], [edge - 3] + [1] * (93 - edge), [20, 1, 69]):
        close(dtype, _run_part(part, session, x, cuts), expected, f"window {window}, cut as {cuts[:4]}...")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_key_that_stands_out_in_latent_attention(dtype):
    """Among 600 keys, those at positions 3 to 12 are made the heaviest for the last ten queries: the key latent's
    matrix repeats the query latent's, head 0's key matrix repeats its query matrix, and each of the last rows repeats
    one of those far rows, so that its query equals that far key (up to the rotated part).  The output must follow it,
    in a prompt and decoded, although no window lets go of anything here."""
    from part_helpers import Session, load_part
    from kirai_b200.weights.random_init import random_tensors

    part, raw = _mixer_part(latent(4, 32, 4, 32, 48, 48, 0.8, scaling=(8.0, 64, 32.0, 1.0)), 96)
    tensors = random_tensors(part.weight_specs(), 21, std=0.08, norm_jitter=0.1, dtype=torch.bfloat16)
    tensors["a.dkv"][:48] = tensors["a.dq"]
    tensors["a.dkv.norm"] = tensors["a.dq.norm"].clone()
    tensors["a.uk"][:32] = tensors["a.uq"][:32]
    w = {k: v.double() for k, v in load_part(part, dtype, seed=21, tensors=tensors).items()}
    x = torch.randn((600, 96), generator=torch.Generator().manual_seed(8))
    x[590:] = x[3:13]
    x = x.to(dtype)
    probabilities = []
    expected = plain.latent_attention(x.double(), w, raw["mixer"], "a.", 1e-5, probabilities)
    far = [float(probabilities[0][590 + i, 3 + i]) for i in range(10)]
    assert min(far) > 0.05 and max(far) > 0.3  # the far keys hold much of head 0's weight (one of 600 evenly: 0.002)
    session = Session([part.cache_need()], dtype, page_size=16, num_pages=80, num_slots=2)
    for cuts in ([600], [570] + [1] * 30, [300, 290, 10]):
        close(dtype, _run_part(part, session, x, cuts), expected, f"cut as {cuts[:3]}...")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_the_gate_stands_between_values_and_output(dtype):
    """A gate matrix scaled until its sigmoid saturates both ways: columns whose gate is shut must vanish ahead of the
    output projection (folding the heads' value matrices into the output projection would let them through)."""
    from part_helpers import Session, load_part
    from kirai_b200.weights.random_init import random_tensors

    part, raw = _mixer_part(latent(4, 8, 8, 16, 24, 16, 1.5), 64)
    tensors = random_tensors(part.weight_specs(), 5, std=0.08, norm_jitter=0.1, dtype=torch.bfloat16)
    tensors["a.g"] = (tensors["a.g"].float() * 40).to(torch.bfloat16)
    w = {k: v.double() for k, v in load_part(part, dtype, seed=5, tensors=tensors).items()}
    x = (torch.randn((30, 64), generator=torch.Generator().manual_seed(4)) * 1.5).to(dtype)
    expected = plain.latent_attention(x.double(), w, raw["mixer"], "a.", 1e-5)
    open_gate = dict(w)
    open_gate["a.g"] = torch.zeros_like(w["a.g"])
    assert float((plain.latent_attention(x.double(), open_gate, raw["mixer"], "a.", 1e-5) * 2 - expected).abs().max()) > 20 * tolerance(dtype, expected.numpy())
    session = Session([part.cache_need()], dtype, page_size=4, num_pages=32, num_slots=2)
    for cuts in ([30], [11, 2] + [1] * 17):
        close(dtype, _run_part(part, session, x, cuts), expected, f"cut as {cuts[:3]}...")


# ------------------------------------------------------------------------ whole models
CLOSE_CALL = 0.02  # a router margin (in scores) below this may fall the other way once activations are rounded to bfloat16


class Reference(np.ndarray):
    """Plain logits [T, vocab] with ``close`` [T]: whether a token's choice of experts, or of open groups, is a close
    call in some layer run.  Such a token is compared in 32-bit only."""


def reference_with_close_calls(config, weights, tokens):
    margins = []
    logits = plain.forward(config, weights, tokens, margins=margins).numpy().view(Reference)
    logits.close = (torch.stack(margins).min(dim=0).values < CLOSE_CALL).numpy() if margins else np.zeros(len(tokens), bool)
    return logits


def check_rows(dtype, got, reference, rows, what):
    expected = np.asarray(reference)[rows]
    assert got.shape == expected.shape, what
    diff = np.abs(got - expected).max(axis=1)
    if dtype in ("bfloat16", torch.bfloat16) and hasattr(reference, "close"):
        diff = np.where(reference.close[rows], 0.0, diff)
    assert float(diff.max()) <= tolerance(dtype, reference), f"{what}: max abs diff {float(diff.max())} (bound {tolerance(dtype, reference)})"


@pytest.fixture(scope="module", params=["A", "B"])
def tiny(request, tmp_path_factory):
    raw, page, seed = TINY[request.param]
    folder = str(tmp_path_factory.mktemp(f"bikilix_{request.param}"))
    write_model(folder, raw, seed)
    config, weights = read_model_folder(folder)
    assert config == raw
    sequences = {rid: random_tokens(n, raw["vocab"], 200 + k)
                 for k, (rid, n) in enumerate([("a", 75), ("b", 40), ("c", 53), ("d", 9), ("e", 61), ("f", 34)])}
    reference = {rid: reference_with_close_calls(config, weights, toks) for rid, toks in sequences.items()}
    return dict(name=request.param, folder=folder, raw=raw, config=config, weights=weights, page=page,
                sequences=sequences, reference=reference)


@pytest.mark.gpu
def test_close_calls_are_few(tiny):
    for rid, reference in tiny["reference"].items():
        assert reference.close.mean() <= 0.5, rid


@pytest.mark.gpu
@pytest.mark.parametrize("fused", ["1", "0"])
def test_residual_stream_after_every_layer_run(tiny, fused, monkeypatch):
    """In 32-bit the stream after each layer run (a looped layer counts each time) equals the plain one, with the norm
    on an output folded into the next norm's kernel and as a kernel of its own."""
    from kirai_b200.engine.batch import StepEntry
    from kirai_b200.engine.runner import ModelRunner
    from kirai_b200.parts.base import NormedSum
    from kirai_b200.parts.block import Block

    monkeypatch.setenv("KIRAI_FUSE_NORMS", fused)
    runner = ModelRunner.from_folder(tiny["folder"], dtype="float32", page_size=tiny["page"], max_tokens=128, num_slots=2)
    tokens = tiny["sequences"]["b"]
    _, streams = plain.forward(tiny["config"], tiny["weights"], tokens, keep_layers=True)
    kept, original, forms = [], Block.forward, set()

    def recording(self, resid, *args, **kwargs):
        stream, left = original(self, resid, *args, **kwargs)
        total = stream.clone()
        forms.add(type(left).__name__)
        if isinstance(left, NormedSum):
            left.settle(total, self.rt.ops)
        kept.append(total.cpu())
        return stream, left

    monkeypatch.setattr(Block, "forward", recording)
    runner.step([StepEntry(runner.cache.open("b"), tokens, [0])])
    assert forms == ({"NormedSum"} if fused == "1" else {"NoneType"})
    assert len(kept) == streams.shape[0] == sum(len(indices) for _, indices in plain.passes(tiny["raw"]))
    for index, stream in enumerate(kept):
        assert float((stream - streams[index]).abs().max()) < 1e-4 * max(1.0, float(streams[index].abs().max())), f"after layer run {index}"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_then_last_tokens_one_by_one(tiny, dtype, tmp_path):
    from replay_client import Replay

    replay = Replay(tiny["folder"], dtype, str(tmp_path / "out"), max_tokens=160, page_size=tiny["page"])
    for rid in ("a", "d"):
        toks = tiny["sequences"][rid]
        got = replay.step([(rid, toks, range(len(toks)))], end=[rid])
        check_rows(dtype, got, tiny["reference"][rid], list(range(len(toks))), f"whole {rid}")
    for rid in ("a", "c"):
        toks = tiny["sequences"][rid]
        head = len(toks) - 40
        got = replay.step([(rid, toks[:head], [0, head - 1])])
        check_rows(dtype, got, tiny["reference"][rid], [0, head - 1], f"{rid} prompt")
        for i in range(head, len(toks)):
            got = replay.step([(rid, [toks[i]], [0])], end=[rid] if i == len(toks) - 1 else [])
            check_rows(dtype, got, tiny["reference"][rid], [i], f"{rid} decode at {i}")
    # a sequence decoded from its very first token
    toks = tiny["sequences"]["f"]
    for i, token in enumerate(toks):
        got = replay.step([("f", [token], [0])], end=["f"] if i == len(toks) - 1 else [])
        check_rows(dtype, got, tiny["reference"]["f"], [i], f"f decode at {i}")
    assert replay.close() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_down_to_two_tokens(tiny, dtype, tmp_path):
    from replay_client import Replay

    replay = Replay(tiny["folder"], dtype, str(tmp_path / "out"), max_tokens=96, page_size=tiny["page"])
    toks = tiny["sequences"]["a"]
    for sizes in ([13, 2, 7, 16, 5, 3, 2, 11, 9, 2, 5], [2] * 37 + [1], [64, 11], [1, 2, 72]):
        assert sum(sizes) == len(toks)
        start = 0
        for size in sizes:
            got = replay.step([("a", toks[start : start + size], range(size))])
            check_rows(dtype, got, tiny["reference"]["a"], list(range(start, start + size)), f"portion at {start}+{size}")
            start += size
        replay.step([], end=["a"])
    assert replay.close() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_on_a_pool_that_runs_full(tiny, dtype, tmp_path):
    """Six unequal requests, at most four live, portions of some beside single tokens of others, on a pool exactly as
    large as the most that live requests hold at once: later requests get pages that earlier ones gave back (the windowed
    layers give pages back as the window passes them), and every logit equals what the request gives alone."""
    from replay_client import Replay
    from test_replay import mixed_schedule, tokens_held_at_most

    sequences, reference, page = tiny["sequences"], tiny["reference"], tiny["page"]
    steps = mixed_schedule(sequences)
    most = tokens_held_at_most(steps, page)
    replay = Replay(tiny["folder"], dtype, str(tmp_path / "out"), max_tokens=most, page_size=page,
                    extra=("--stats", str(tmp_path / "out" / "stats.json"), "--max-requests", "4"))
    for entries, end in steps:
        batch = [(rid, sequences[rid][first : first + count], range(count)) for rid, first, count in entries]
        got = replay.step(batch, end=end)
        row = 0
        for rid, first, count in entries:
            check_rows(dtype, got[row : row + count], reference[rid], list(range(first, first + count)), f"mixed {rid} at {first}+{count}")
            row += count
    assert replay.close() == 0
    stats = replay.stats()
    assert stats["live_requests"] == 0
    assert all(group["used"] == 0 and group["pages"] >= group["high_water"] > 0 for group in stats["groups"])
    assert any(group["high_water"] == group["pages"] == most // page < group["handed_out"] for group in stats["groups"])


# C: sizes of a small real model, on which bfloat16 takes the tensor-core kernels: heads of 64 in a group of 4 (the
# tcgen05 prompt kernel, the decode kernels), heads of 128 in a group of 3 with narrower values, a latent row of 128 and
# one of 256 columns, windows of 100 and 64 tokens on pages of 16, experts of 128 on a width of 256 (rows sorted by
# expert for long portions), a stretch that runs twice with a layer behind it.
CONFIG_C = {
    "architecture": "Bikilix", "width": 256, "vocab": 320, "norm": {"eps": 1e-6}, "embedding": {"scale": 4.0},
    "layers": [
        layer(attn(8, 2, 64, 64, 0.9, rot(10000.0, 32), 100), dense(384)),
        layer(latent(8, 32, 32, 32, 96, 96, 0.7, scaling=(8.0, 128, 32.0, 1.0)), moe(128, 1.2, 8, 2, 4, 2)),
        layer(latent(4, 64, 64, 64, 128, 192, 0.5), dense(256)),
        layer(attn(6, 2, 128, 64, 0.6, rot(50000.0, 128), 64), moe(128, 0.8, 6, 3, 3, 2)),
    ],
    "loop": {"start": 0, "stop": 3, "times": 2},
}


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompts_whole_in_portions_and_beside_decoded_tokens(dtype, tmp_path):
    from replay_client import Replay

    folder = str(tmp_path / "model")
    write_model(folder, CONFIG_C, 31, std=0.05)
    config, weights = read_model_folder(folder)
    long_a, long_b = random_tokens(650, 320, 1), random_tokens(420, 320, 2)
    ref_a, ref_b = reference_with_close_calls(config, weights, long_a), reference_with_close_calls(config, weights, long_b)
    assert ref_a.close.mean() < 0.5 and ref_b.close.mean() < 0.5
    replay = Replay(folder, dtype, str(tmp_path / "out"), max_tokens=1200, page_size=16)
    want = [0, 63, 64, 99, 100, 101, 163, 164, 199, 200, 399, 400, 511, 512, 600, 649]
    got = replay.step([("a", long_a, want)], end=["a"])
    check_rows(dtype, got, ref_a, want, "whole")
    start = 0
    for size in (300, 2, 97, 1, 113, 87, 50):
        rows = sorted({0, size - 1, size // 2})
        got = replay.step([("a", long_a[start : start + size], rows)])
        check_rows(dtype, got, ref_a, [start + r for r in rows], f"portion at {start}+{size}")
        start += size
    assert start == 650
    # b's prompt in one portion, then b decoding beside a second run of a's prompt
    got = replay.step([("b", long_b[:390], [389])], end=["a"])
    check_rows(dtype, got, ref_b, [389], "b prompt")
    position, a_at = 390, 0
    for size in (128, 2, 200, 1, 64, 255):
        entries = [("a2", long_a[a_at : a_at + size], [size - 1])]
        if position < 420:
            entries.append(("b", [long_b[position]], [0]))
        got = replay.step(entries)
        check_rows(dtype, got[:1], ref_a, [a_at + size - 1], f"a beside b at {a_at}+{size}")
        if position < 420:
            check_rows(dtype, got[1:], ref_b, [position], f"b decode at {position}")
            position += 1
        a_at += size
    while position < 420:
        got = replay.step([("b", [long_b[position]], [0])])
        check_rows(dtype, got, ref_b, [position], f"b decode at {position}")
        position += 1
    assert replay.close() == 0


def random_configuration(seed, wide=False):
    """A configuration drawn from sizes that are and are not multiples of 8, any order and number of layers, layers
    without feed-forward, both feed-forwards, with and without stretched frequencies, a loop over any stretch or none.
    ``wide``: heads and latent rows of up to 256 columns, which the tensor-core kernels take in other forms."""
    import random

    r = random.Random(seed + (1000 if wide else 0))
    width = r.choice([32, 40, 72, 96, 130])
    layers = []
    for _ in range(r.randint(2, 5)):
        if r.random() < 0.5:
            kv_heads, dim = r.choice([1, 2, 3, 4]), r.choice([96, 128, 136, 200, 256] if wide else [8, 12, 16, 24, 32, 40, 64])
            dims = r.choice([d for d in (2, 4, 6, 8, 16, 32, 64) if d <= dim] + [dim])
            entry = attn(kv_heads * r.choice([1, 2, 3, 4, 5, 8]), kv_heads, dim, r.choice([64, 128, 160, 256] if wide else [8, 12, 16, 24, 32, 40, 64]),
                         r.uniform(0.5, 1.5) * 4 / dim ** 0.5, rot(r.choice([50.0, 10000.0, 1e6]), dims),
                         r.choice([None, 1, 3, 7, 16, 33, 64, 200]))
        else:
            rot_dim = r.choice([2, 4, 6, 8, 16, 32])
            scaling = r.choice([None, (r.choice([2.0, 8.0, 40.0]), r.choice([8, 16, 64]), r.choice([4.0, 32.0]), r.choice([0.5, 1.0]))])
            entry = latent(r.choice([1, 2, 4, 6, 8, 20]), r.choice([4, 8, 10, 16, 32]), rot_dim, r.choice([4, 8, 12, 16]),
                           r.choice([8, 20, 24, 48]), r.choice([100, 128, 192, 224] if wide else [6, 16, 18, 32, 64]), r.uniform(0.5, 1.5),
                           base=r.choice([100.0, 10000.0]), scaling=scaling)
        kind = r.choice(["none", "dense", "moe", "moe"])
        if kind == "moe":
            count = r.choice([1, 2, 3, 4])
            size = r.choice([1, 2, 3, 5])
            keep = r.randint(1, count)
            mlp = moe(r.choice([4, 8, 12, 20]), r.choice([0.3, 1.0, 7.0]), count * size, r.randint(1, min(4, keep * size)), count, keep)
        else:
            mlp = None if kind == "none" else dense(r.choice([16, 36, 52, 96]))
        layers.append(layer(entry, mlp))
    raw = {"architecture": "Bikilix", "width": width, "vocab": r.choice([50, 97, 260]), "norm": {"eps": r.choice([1e-6, 1e-5, 1e-3])},
           "embedding": {"scale": r.choice([0.5, 1.0, 3.0])}, "layers": layers}
    if r.random() < 0.7:
        start = r.randrange(len(layers))
        raw["loop"] = {"start": start, "stop": r.randint(start + 1, len(layers)), "times": r.randint(1, 3)}
    return raw, r.choice([4, 8, 16, 16])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", list(range(8)) + [-1, -2, -3, -4])
def test_random_configurations_whole_in_portions_and_mixed(seed, dtype, tmp_path):
    """Three requests of a randomly drawn configuration: one whole, one in portions with its last tokens one by one,
    and all three side by side in unequal runs, on pages that are given back and used again."""
    from kirai_b200.engine.batch import StepEntry
    from kirai_b200.engine.runner import ModelRunner

    raw, page = random_configuration(abs(seed), wide=seed < 0)  # negative seeds draw wide heads and rows
    folder = str(tmp_path / "model")
    write_model(folder, raw, 100 + seed, std=0.05 if seed < 0 else 0.08)
    config, weights = read_model_folder(folder)
    sequences = {rid: random_tokens(n, raw["vocab"], 300 + seed + k) for k, (rid, n) in enumerate([("a", 83), ("b", 37), ("c", 58)])}
    reference = {rid: reference_with_close_calls(config, weights, toks) for rid, toks in sequences.items()}
    bound = {rid: (3e-5 * max(1.0, float(np.abs(ref).max())) if dtype == "float32" else 0.07 * float(np.abs(ref).max()))
             for rid, ref in reference.items()}
    runner = ModelRunner.from_folder(folder, dtype=dtype, page_size=page, max_tokens=3 * 96, num_slots=4)
    whole = {}  # every request alone and whole through the framework: what any other schedule must give, up to rounding
    for rid, toks in sequences.items():
        request = runner.cache.open((rid, "whole"))
        whole[rid] = runner.step([StepEntry(request, toks, list(range(len(toks))))]).cpu().numpy()
        runner.cache.close(request)

    def run(steps):
        live, done = {}, {rid: 0 for rid in sequences}
        for step in steps:
            entries, names = [], []
            for rid, count in step:
                if rid not in live:
                    live[rid] = runner.cache.open((rid, id(steps)))
                tokens = sequences[rid][done[rid] : done[rid] + count]
                entries.append(StepEntry(live[rid], tokens, list(range(count))))
                names.append((rid, done[rid], count))
                done[rid] += count
            logits = runner.step(entries).cpu().numpy()
            row = 0
            for rid, first, count in names:
                diff = np.abs(logits[row : row + count] - np.asarray(reference[rid])[first : first + count]).max(axis=1)
                if dtype == "bfloat16":
                    diff = np.where(reference[rid].close[first : first + count], 0.0, diff)
                assert float(diff.max()) <= bound[rid], f"{raw}: {rid} at {first}+{count}: max abs diff {float(diff.max())} (bound {bound[rid]})"
                own = np.abs(logits[row : row + count] - whole[rid][first : first + count]).max(axis=1)
                if dtype == "bfloat16":
                    own = np.where(reference[rid].close[first : first + count], 0.0, own)
                assert float(own.max()) <= 0.6 * bound[rid], f"{raw}: {rid} at {first}+{count} against its whole run: {float(own.max())}"
                row += count
        for request in live.values():
            runner.cache.close(request)

    run([[("a", 83)]])
    run([[("b", 9)], [("b", 2)], [("b", 16)], [("b", 5)]] + [[("b", 1)]] * 5)
    run([[("a", 30), ("c", 1)], [("c", 1), ("b", 20)], [("a", 1), ("b", 1), ("c", 40)], [("a", 52), ("b", 16), ("c", 16)]])
    run([[("c", 58), ("a", 2)], [("a", 81), ("b", 37)]])


# ---------------------------------------------------------------------- generation
def _plain_greedy(config, weights, prompt, count):
    tokens = list(prompt)
    for _ in range(count):
        logits = plain.forward(config, weights, tokens)[-1]
        tokens.append(int(torch.nonzero(logits == logits.max())[0]))
    return tokens[len(prompt):]


def _sure(config, weights, prompt, generated):
    """Whether the plain greedy tokens are safe from rounding: no close call among the experts, no two logits near a tie."""
    margins = []
    logits = plain.forward(config, weights, list(prompt) + list(generated), margins=margins)
    top2 = torch.topk(logits[len(prompt) - 1 : -1], 2, dim=-1).values
    calls = float(torch.stack(margins).min()) if margins else 1.0
    return bool(((top2[:, 0] - top2[:, 1]) > 4 * tolerance("bfloat16", logits.numpy())).all()) and calls > CLOSE_CALL


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(tiny, dtype):
    """Five prompts through the scheduler (three at a time, prompts in portions of 16, decode steps from captured graphs
    where the engine captures them) give the plain implementation's greedy tokens."""
    from kirai_b200 import Engine, SamplingParams

    engine = Engine(tiny["folder"], dtype=dtype, page_size=tiny["page"], max_prefill_tokens=16, max_concurrent_requests=3,
                    max_new_tokens=16, max_cache_tokens=256)
    prompts = [random_tokens(n, tiny["raw"]["vocab"], 50 + n) for n in (5, 11, 17, 3, 24)]
    outputs = engine.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=8))
    compared = 0
    for prompt, output in zip(prompts, outputs):
        expected = _plain_greedy(tiny["config"], tiny["weights"], prompt, 8)
        assert output.finish_reason == "length" and (output.prompt_tokens, output.completion_tokens) == (len(prompt), 8)
        if dtype == "float32" or _sure(tiny["config"], tiny["weights"], prompt, expected):
            assert output.token_ids == expected
            compared += 1
    assert compared >= (5 if dtype == "float32" else 0)
    stats = engine.stats()
    assert stats["cache"]["live_requests"] == 0 and all(g["used"] == 0 for g in stats["cache"]["groups"])
    assert engine.runner.model.plan.capture_safe()


@pytest.mark.gpu
def test_long_decoding_through_captured_steps_follows_the_plain_model(tiny):
    """One request decodes 70 tokens in 32-bit: past the windows, across many pages, every pass of the loop with its own
    cache; the tokens equal the plain implementation's, which sees the whole sequence at once."""
    from kirai_b200 import Engine, SamplingParams

    engine = Engine(tiny["folder"], dtype="float32", page_size=tiny["page"], max_new_tokens=80, max_cache_tokens=256)
    prompt = random_tokens(7, tiny["raw"]["vocab"], 5)
    output = engine.generate([prompt], SamplingParams(temperature=0.0, max_new_tokens=70))[0]
    logits = plain.forward(tiny["config"], tiny["weights"], list(prompt) + output.token_ids)[len(prompt) - 1 : -1]
    chosen = logits[torch.arange(70), torch.tensor(output.token_ids)]
    assert bool((chosen >= logits.max(dim=-1).values - 1e-4).all())


@pytest.mark.gpu
def test_eviction_and_recompute_give_the_same_sampled_tokens(tiny):
    from kirai_b200 import Engine, SamplingParams

    params = SamplingParams(temperature=0.8, top_p=0.95, seed=5, max_new_tokens=14)
    prompts = [random_tokens(17, tiny["raw"]["vocab"], 1), random_tokens(18, tiny["raw"]["vocab"], 2)]
    roomy = Engine(tiny["folder"], dtype="float32", page_size=tiny["page"], max_new_tokens=16, max_cache_tokens=256)
    expected = [o.token_ids for o in roomy.generate(prompts, params)]
    tight = Engine(tiny["folder"], dtype="float32", page_size=tiny["page"], max_new_tokens=16, max_cache_tokens=48)
    outputs = tight.generate(prompts, params)
    assert [o.token_ids for o in outputs] == expected
    assert tight.stats()["scheduler"]["preemptions"] >= 1 and sum(o.preemptions for o in outputs) >= 1


@pytest.mark.gpu
def test_command_line_generates(tiny):
    prompt = random_tokens(9, tiny["raw"]["vocab"], 77)
    result = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "kirai"), "generate", "--snapshot", tiny["folder"],
                             "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "6", "--temperature", "0",
                             "--dtype", "float32", "--page-size", str(tiny["page"])], capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr
    expected = _plain_greedy(tiny["config"], tiny["weights"], prompt, 6)
    assert json.loads(result.stdout.strip().splitlines()[-1])["token_ids"] == expected
