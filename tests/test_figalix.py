"""The Figalix decoder against a plain implementation written from the design's equations (``plain_figalix``):
each mechanism alone, whole models whole, in portions, decoded, mixed, and generation through the engine.

Tiny configurations and random weights are made here; where random weights would hide a fault (a window's edge, the
kept first keys, a far key, the cap on a gate) rows or weights are scaled so that it shows.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_figalix as plain
from plain_qwen3 import read_model_folder
from tiny_configs import random_tokens

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = [torch.float32, torch.bfloat16]


def rot(base, dims, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling:
        out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return out


def attn(heads, kv_heads, dim, vdim, scale, rotation, size, keep_first):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rotation,
            "mask": {"size": size, "keep_first": keep_first}}


def memory(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def parallel(left, right):
    return {"type": "parallel", "mixer": {"left": left, "right": right}}


def mamba(heads, vdim, state, groups, conv, norm_groups):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def layer(entry, mlp):
    return {**entry, "mlp": mlp}


# A: sizes in multiples of 8; a window of two pages that keeps three first keys; a stretched rotation of half a
# head; an attention side whose window keeps nothing and whose heads are rotated whole; a state-space layer without
# feed-forward; experts with and without a shared branch.  B: nothing a multiple of 8, six query heads on one kv head,
# more kept keys than the window is wide, a convolution of one tap (no kept rows), as many groups as heads, every
# expert chosen, no factor on the sub-layers (1) and a parallel layer first.
CONFIG_A = {
    "architecture": "Figalix", "width": 64, "vocab": 200, "norm": {"eps": 1e-5}, "residual_mult": 0.5, "logit_softcap": 6.0,
    "layers": [
        layer(mamba(4, 8, 16, 2, 4, 2), dense(96)),
        layer(parallel(attn(4, 2, 16, 16, 0.7, rot(500.0, 8, (4.0, 32, 4.0, 1.0)), 8, 3), memory(2, 8, 16, 5.0)), moe(4, 2, 24, 16)),
        layer(mamba(2, 16, 8, 1, 2, 1), None),
        layer(parallel(attn(2, 2, 32, 8, 0.4, rot(10000.0, 32), 16, 0), memory(4, 4, 4, 15.0)), moe(3, 1, 16)),
    ],
}
CONFIG_B = {
    "architecture": "Figalix", "width": 100, "vocab": 131, "norm": {"eps": 1e-3}, "residual_mult": 1.0, "logit_softcap": 30.0,
    "layers": [
        layer(parallel(attn(6, 1, 12, 20, 0.9, rot(77.0, 4, (2.0, 16, 3.0, 0.5)), 5, 7), memory(3, 10, 12, 2.0)), dense(52)),
        layer(mamba(5, 12, 6, 5, 3, 3), moe(5, 3, 20, 28)),
        layer(mamba(3, 20, 24, 1, 1, 1), None),
        layer(parallel(attn(3, 3, 10, 6, 1.1, rot(50.0, 10), 11, 1), memory(1, 24, 20, 8.0)), moe(2, 2, 12, 8)),
    ],
}
TINY = {"A": (CONFIG_A, 4, 3), "B": (CONFIG_B, 8, 4)}  # name -> (config, page size, seed)


def write_model(folder, raw, seed, std=0.08):
    import kirai_b200  # noqa: F401
    from kirai_b200.registry import config_from_dict
    from kirai_b200.weights import write_random_model

    write_random_model(folder, config_from_dict(raw), seed, std=std, norm_jitter=0.3, dtype=torch.bfloat16)


def tolerance(dtype, reference):
    dtype = {torch.float32: "float32", torch.bfloat16: "bfloat16"}.get(dtype, dtype)
    peak = float(np.abs(np.asarray(reference)).max())
    return 3e-5 * max(1.0, peak) if dtype == "float32" else 0.035 * peak


def close(dtype, got, expected, what, rows=None):
    got, expected = np.asarray(got, dtype=np.float64), np.asarray(expected, dtype=np.float64)
    assert got.shape == expected.shape, what
    diff = np.abs(got - expected)
    if rows is not None:
        diff = diff[rows]
    worst = float(diff.max()) if diff.size else 0.0
    assert worst <= tolerance(dtype, expected), f"{what}: max abs diff {worst} (bound {tolerance(dtype, expected)})"


# --------------------------------------------------------------------------- no GPU
def test_config_reads_every_size_and_round_trips():
    import kirai_b200  # noqa: F401
    from kirai_b200.config.base import ConfigError
    from kirai_b200.parts.base import KVCacheNeed, StateNeed
    from kirai_b200.registry import config_from_dict, plan_for_config

    for raw in (CONFIG_A, CONFIG_B):
        cfg = config_from_dict(raw)
        assert cfg.to_dict() == raw and config_from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
        plan = plan_for_config(cfg)
        needs = plan.cache_needs
        at = 0
        for entry in raw["layers"]:
            m = entry["mixer"]
            if entry["type"] == "parallel":
                kv, state = needs[at], needs[at + 1]
                assert isinstance(kv, KVCacheNeed) and isinstance(state, StateNeed)
                left, right = m["left"], m["right"]
                assert (kv.kv_heads, kv.window, kv.keep_first) == (left["kv_heads"], left["mask"]["size"], left["mask"]["keep_first"])
                assert (kv.key_dim or kv.head_dim, kv.value_dim or kv.head_dim) == (left["dim"], left["vdim"])
                assert state.shape == (right["heads"] * (right["dim"] * right["vdim"] + right["dim"] + 1),)
                at += 2
            else:
                channels = m["heads"] * m["vdim"] + 2 * m["groups"] * m["state"]
                assert needs[at].shape == ((m["conv"] - 1) * channels + m["heads"] * m["state"] * m["vdim"],)
                assert needs[at].dtype == torch.float32
                at += 1
        assert at == len(needs)
        names = set(plan.weight_specs())
        assert {"embed", "final.norm", "final.norm.alpha", "final.norm.b", "l0.norm1.alpha"} <= names
        assert not any(name.startswith("l2.mlp") or name.startswith("l2.norm2") for name in names)  # no feed-forward there
    bad = json.loads(json.dumps(CONFIG_A))
    bad["layers"][0]["type"] = "conv"
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = json.loads(json.dumps(CONFIG_A))
    bad["layers"][1]["mixer"]["left"]["kv_heads"] = 3
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = json.loads(json.dumps(CONFIG_A))
    bad["layers"][0]["mixer"]["norm_groups"] = 3
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = json.loads(json.dumps(CONFIG_A))
    bad["layers"][1]["mlp"]["router"]["top"] = 5
    with pytest.raises(ConfigError):
        config_from_dict(bad)


def test_frequencies_stretched_by_index():
    """The framework's table equals the plain one; the ramp leaves fast frequencies alone, divides slow ones by the
    factor, and the amplitude is 0.1 ln(factor) + 1."""
    import math

    from kirai_b200.parts.rope import RotaryEmbedding

    for base, dims, scaling in ((500.0, 8, (4.0, 32, 4.0, 1.0)), (77.0, 4, (2.0, 16, 3.0, 0.5)), (1e4, 64, (16.0, 4096, 32.0, 1.0)),
                                (1e6, 32, (8.0, 128, 2.0, 2.0)), (1e4, 16, None)):
        raw = rot(base, dims, scaling)
        expected, amplitude = plain.stretched_frequencies(raw)
        part = RotaryEmbedding(dims + 8, base, dims, scaling=raw.get("scaling"), precise=True)
        assert torch.allclose(part.frequencies().double(), expected, rtol=1e-6, atol=0.0)
        assert abs(part.amplitude - amplitude) < 1e-12
        plain_f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
        if scaling:
            assert abs(amplitude - (0.1 * math.log(scaling[0]) + 1.0)) < 1e-12
            ratio = expected / plain_f
            assert float(ratio.max()) <= 1.0 + 1e-12 and float(ratio.min()) >= 1.0 / scaling[0] - 1e-12
            assert all(float(ratio[i]) >= float(ratio[i + 1]) - 1e-12 for i in range(len(ratio) - 1))
        else:
            assert amplitude == 1.0 and torch.equal(expected, plain_f)
    stretched, _ = plain.stretched_frequencies(rot(1e4, 64, (16.0, 4096, 32.0, 1.0)))
    plain_f = torch.tensor([1e4 ** (-2.0 * i / 64) for i in range(32)], dtype=torch.float64)
    assert float(stretched[0]) == float(plain_f[0]) and abs(float(stretched[-1]) * 16.0 / float(plain_f[-1]) - 1.0) < 1e-12


def test_plain_mask_and_page_tables_keep_the_first_keys():
    """Row i of the mask sees j <= i with i - j < size or j < keep_first; both page tables hold on to the pages of the
    kept keys while the window gives the others back."""
    see = plain.visible_keys(12, 4, 2)
    assert see[11].tolist() == [True, True] + [False] * 6 + [True] * 4
    assert see[3].tolist() == [True] * 4 + [False] * 8 and see[5].tolist() == [True, True, True, True, True, True] + [False] * 6
    assert plain.visible_keys(6, 2, 0)[5].tolist() == [False] * 4 + [True] * 2
    from kirai_b200.cache.native_pages import NativePageTables
    from kirai_b200.cache.pages import NO_PAGE, GroupSpec, PageTables

    for tables_class in (PageTables, NativePageTables):
        tables = tables_class([GroupSpec(1, 8, 6, keep_first=5), GroupSpec(1, 8, 6)], 4, [16, 16], 2)
        request = tables.open("r")
        for count in (9, 1, 1, 14, 3):
            assert tables.reserve(request, count)
            tables.commit(request, count)
        kept, plain_window = (list(tables.fill_tables([request], g, 1)[0]) if tables_class is NativePageTables
                              else list(request.tables[g]) for g in (0, 1))
        # 28 tokens, the first visible key of the next position is 23: pages 0 to 4 lie wholly before it
        assert [p != NO_PAGE for p in kept] == [True, True, False, False, False, True, True]
        assert [p != NO_PAGE for p in plain_window] == [False] * 5 + [True, True]
        tables.close(request)
        assert all(pool.free_pages == 16 for pool in tables.pools)


# ------------------------------------------------------------------------ parts alone
def _mixer(entry, width, eps=1e-5):
    """The framework's mixer of one configured layer (its tensors under ``a.``) and the layer as config.json holds it."""
    import kirai_b200  # noqa: F401
    from kirai_b200.config.figalix import FigalixConfig
    from kirai_b200.models.figalix import mixer_for_layer

    raw = {"architecture": "Figalix", "width": width, "vocab": 8, "norm": {"eps": eps}, "residual_mult": 1.0,
           "layers": [layer(entry, None)]}
    cfg = FigalixConfig.from_dict(raw)
    return mixer_for_layer(cfg, cfg.layers[0], "a."), raw["layers"][0]["mixer"]


def _needs(part):
    need = part.cache_need()
    return list(need) if isinstance(need, tuple) else [need]


def _view(part, session):
    if isinstance(part.cache_need(), tuple):
        return tuple(session.cache.layer_view(i) for i in range(len(part.cache_need())))
    return session.cache.layer_view(0)


def _run_together(part, session, xs, steps):
    """The part's output rows for several requests (``xs``: name -> rows [T, width]) under a schedule: ``steps`` is a
    list of steps, each a list of (name, count) that run as one batch.  A request is closed after its last row."""
    names = list(xs)
    offset, table = {}, []
    for name in names:
        offset[name] = sum(t.shape[0] for t in table)
        table.append(xs[name])
    table = torch.cat(table)
    done = {name: 0 for name in names}
    out = None
    for step in steps:
        runs = [(name, list(range(offset[name] + done[name], offset[name] + done[name] + count))) for name, count in step]
        batch = session.batch(runs)
        rows = batch.token_ids.cpu().long()
        y = part.forward(table[rows].cuda(), batch, _view(part, session)).float().cpu()
        if out is None:
            out = torch.zeros((table.shape[0], y.shape[1]))
        out[rows] = y
        session.commit()
        for name, count in step:
            done[name] += count
            if done[name] == xs[name].shape[0]:
                session.cache.close(session.requests.pop(name))
    assert all(done[name] == xs[name].shape[0] for name in names)
    return {name: out[offset[name] : offset[name] + xs[name].shape[0]] for name in names}


def _run_part(part, session, x, cuts):
    return _run_together(part, session, {"s": x}, [[("s", size)] for size in cuts])["s"]


CUTS = lambda n: ([n], [37, 2, 19, 1, 1, 3, n - 63], [n - 10] + [1] * 10, [2] * (n // 2) + [1] * (n % 2), [1] * n)  # noqa: E731


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [64, 100, 7, 2048 + 24])
def test_dynamic_tanh_with_a_scaled_sum_and_chosen_rows(dtype, width):
    from part_helpers import load_part
    from kirai_b200.parts import DynamicTanh
    from kirai_b200.parts.base import ScaledSum

    norm = DynamicTanh("n", width)
    w = load_part(norm, dtype, seed=width)
    g = torch.Generator().manual_seed(width)
    stream, d1, d2 = (torch.randn((11, width), generator=g) * s for s in (2.0, 1.0, 0.5))

    def expected(x):
        return torch.tanh(w["n.alpha"].double() * x.double()) * w["n"].double() + w["n.b"].double()

    for terms, factor in (([], 1.0), ([d1], 0.37), ([d1, d2], 1.5)):
        resid = stream.clone().cuda()
        delta = ScaledSum([t.cuda() for t in terms], factor) if terms else None
        out = norm.add_forward(resid, delta)
        total = stream.double() + factor * sum(t.double() for t in terms) if terms else stream.double()
        assert out.dtype == dtype and float((resid.cpu().double() - total).abs().max()) < 1e-5
        close(dtype, out.float().cpu(), expected(total), f"{len(terms)} terms")
        rows = torch.tensor([9, 0, 4], dtype=torch.int32)
        resid = stream.clone().cuda()
        picked = norm.add_forward_rows(resid, delta, rows.cuda())
        assert torch.equal(resid.cpu(), stream)  # chosen rows leave the stream alone
        close(dtype, picked.float().cpu(), expected(total)[rows.long()], "chosen rows")


@pytest.mark.gpu
@pytest.mark.parametrize("width", [64, 100, 7, 1024 + 40])
def test_mean_of_two_unit_rms_rows(width):
    from kirai_b200.csrc import ops

    g = torch.Generator().manual_seed(width)
    a, b = torch.randn((9, width), generator=g) * 3.0, torch.randn((9, width), generator=g) * 0.01
    wa, wb = torch.randn(width, generator=g), torch.randn(width, generator=g)
    for eps in (1e-6, 1e-2):
        got = ops.rms_pair_mean(a.cuda(), b.cuda(), wa.cuda(), wb.cuda(), eps).cpu()
        expected = 0.5 * (plain.unit_rms(a.double(), eps) * wa.double() + plain.unit_rms(b.double(), eps) * wb.double())
        close(torch.float32, got, expected, f"eps {eps}")


STATE_SPACE_CASES = [  # heads, vdim, state, groups, taps, norm groups, width
    (4, 8, 16, 2, 4, 2, 64), (5, 12, 6, 5, 3, 3, 100), (3, 20, 24, 1, 1, 1, 40), (2, 64, 128, 1, 4, 4, 96), (8, 32, 48, 2, 2, 1, 72),
    (1, 7, 3, 1, 5, 1, 24), (6, 16, 256, 3, 4, 2, 64),
]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", STATE_SPACE_CASES, ids=lambda c: "x".join(map(str, c)))
def test_state_space_whole_in_portions_and_one_by_one(dtype, case):
    """The convolution's kept rows and the heads' states carry from step to step, start at zero in a slot that an
    earlier request used, and every cut of the rows gives the plain result."""
    from part_helpers import Session, load_part

    *sizes, width = case
    part, raw = _mixer(mamba(*sizes), width)
    w = {k: v.double() for k, v in load_part(part, dtype, seed=sum(case)).items()}
    tokens = 90
    x = (torch.randn((tokens, width), generator=torch.Generator().manual_seed(width)) * 1.5).to(dtype)
    expected = plain.state_space(x.double(), w, raw, "a.", 1e-5)
    session = Session(_needs(part), dtype, page_size=4, num_pages=4, num_slots=2)
    for cuts in CUTS(tokens):
        close(dtype, _run_part(part, session, x, cuts), expected, f"cut as {cuts[:4]}...")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_state_space_decays_and_step_sizes_show(dtype):
    """With A_log and dt_bias spread wide (decays from almost 1 to almost 0, step sizes from 0.01 to 6: softplus has no
    clamp) a long decoding still follows the plain recurrence, and a state that forgot nothing differs from one that
    forgot everything."""
    from part_helpers import Session, load_part
    from kirai_b200.weights.random_init import random_tensors

    part, raw = _mixer(mamba(4, 16, 32, 2, 4, 1), 64)
    tensors = random_tensors(part.weight_specs(), 5, std=0.08, norm_jitter=0.1, dtype=torch.bfloat16)
    tensors["a.A_log"] = torch.tensor([-6.0, -1.0, 0.5, 2.0]).to(torch.bfloat16)
    tensors["a.dt_bias"] = torch.tensor([-4.5, 0.0, 2.0, 6.0]).to(torch.bfloat16)
    w = {k: v.double() for k, v in load_part(part, dtype, seed=5, tensors=tensors).items()}
    x = (torch.randn((300, 64), generator=torch.Generator().manual_seed(3)) * 1.5).to(dtype)
    expected = plain.state_space(x.double(), w, raw, "a.", 1e-5)
    session = Session(_needs(part), dtype, page_size=4, num_pages=4, num_slots=2)
    for cuts in ([300], [10] + [1] * 290, [150, 75, 75]):
        close(dtype, _run_part(part, session, x, cuts), expected, f"cut as {cuts[:3]}...")


MEMORY_CASES = [  # heads, dim, vdim, cap, width
    (2, 8, 16, 5.0, 64), (3, 10, 12, 2.0, 100), (1, 24, 20, 8.0, 40), (4, 64, 128, 15.0, 96), (4, 4, 4, 15.0, 24), (2, 128, 64, 10.0, 64),
    (1, 256, 32, 4.0, 48),
]


def _memory_part(case):
    from kirai_b200.parts import MatrixMemory

    heads, dim, vdim, cap, width = case
    return MatrixMemory("a.", width, heads, dim, vdim, cap, 1e-5, out_dtype=torch.float32), memory(heads, dim, vdim, cap)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", MEMORY_CASES, ids=lambda c: "x".join(map(str, c)))
def test_matrix_memory_whole_in_portions_and_one_by_one(dtype, case):
    from part_helpers import Session, load_part
    from kirai_b200.weights.random_init import random_tensors

    part, raw = _memory_part(case)
    tensors = random_tensors(part.weight_specs(), sum(map(int, case)), std=0.08, norm_jitter=0.1, dtype=torch.bfloat16)
    # gates that reach the cap on both sides, and a forget gate that forgets: the running maximum moves both ways
    tensors["a.i"] *= 12.0
    tensors["a.f"] *= 12.0
    tensors["a.i.b"] = torch.linspace(-2.0, 3.0, case[0]).to(torch.bfloat16)
    tensors["a.f.b"] = torch.linspace(2.0, -1.0, case[0]).to(torch.bfloat16)
    w = {k: v.double() for k, v in load_part(part, dtype, seed=0, tensors=tensors).items()}
    tokens = 90
    x = (torch.randn((tokens, case[-1]), generator=torch.Generator().manual_seed(case[1])) * 1.5).to(dtype)
    expected = plain.matrix_memory(x.double(), w, raw, "a.", 1e-5)
    uncapped = plain.matrix_memory(x.double(), w, {**raw, "gate_cap": 1e6}, "a.", 1e-5)
    assert float((uncapped - expected).abs().max()) > 3 * tolerance(dtype, expected.numpy())  # the cap matters here
    session = Session(_needs(part), dtype, page_size=4, num_pages=4, num_slots=2)
    for cuts in CUTS(tokens):
        close(dtype, _run_part(part, session, x, cuts), expected, f"cut as {cuts[:4]}...")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_matrix_memory_first_tokens_and_long_decoding(dtype):
    """Input gates far below zero, so that the running maximum stays where it starts (at 0) for the first tokens and the
    read-out's lower bound exp(-m) holds; forget gates that keep almost everything in one head and forget in the
    other.  Whole, 400 tokens one by one, and in large portions."""
    from part_helpers import Session, load_part
    from kirai_b200.weights.random_init import random_tensors

    part, raw = _memory_part((2, 16, 16, 12.0, 48))
    tensors = random_tensors(part.weight_specs(), 77, std=0.08, norm_jitter=0.1, dtype=torch.bfloat16)
    tensors["a.i.b"] = torch.tensor([-9.0, -6.0]).to(torch.bfloat16)
    tensors["a.f.b"] = torch.tensor([4.0, 1.0]).to(torch.bfloat16)
    w = {k: v.double() for k, v in load_part(part, dtype, seed=0, tensors=tensors).items()}
    x = (torch.randn((400, 48), generator=torch.Generator().manual_seed(6)) * 1.5).to(dtype)
    expected = plain.matrix_memory(x.double(), w, raw, "a.", 1e-5)
    session = Session(_needs(part), dtype, page_size=4, num_pages=4, num_slots=2)
    for cuts in ([400], [1] * 400, [3, 200, 197]):
        close(dtype, _run_part(part, session, x, cuts), expected, f"cut as {cuts[:3]}...")


# the three forms of a step's runs through a matrix state: chunks one after another in a block, chunks side by side with
# a carry between them, and token by token
FORMS = (dict(chain_limit=10 ** 9), dict(chain_limit=0), dict(walk_limit=10 ** 9))


def _plain_scan(q, k, v, keep_log, take_log, take_scale, S, n, m, floor):
    """One head's recurrence over rows, in 64-bit and token by token.  ``floor``: the read-out is divided by
    max(|n . q|, exp(-m)) + 1e-6 and a running maximum is kept (the matrix memory); else neither (the state space)."""
    out = []
    for t in range(q.shape[0]):
        if floor:
            m_new = max(keep_log[t] + m, take_log[t])
            keep, take = np.exp(keep_log[t] + m - m_new), np.exp(take_log[t] - m_new)
            m = m_new
        else:
            keep, take = np.exp(keep_log[t]), take_scale[t]
        S = keep * S + take * np.outer(k[t], v[t])
        n = keep * n + take * k[t]
        o = S.T @ q[t]
        out.append(o / (max(abs(float(n @ q[t])), np.exp(-m)) + 1e-6) if floor else o)
    return np.stack(out), S, n, m


@pytest.mark.gpu
@pytest.mark.parametrize("heads,groups,state,vdim", [(4, 2, 16, 8), (3, 3, 40, 20), (2, 1, 128, 64), (2, 1, 256, 80), (1, 1, 5, 3)])
def test_state_space_runs_in_chunks_as_token_by_token(heads, groups, state, vdim):
    """Unequal requests in one step (a run shorter than a chunk, one of a chunk exactly, one of a chunk and a token,
    one of several chunks, a single token) from states that are not zero: the chunked kernels (both forms), the walk and a plain
    loop agree on the outputs and on the states they leave."""
    from part_helpers import Session
    from kirai_b200.parts.base import StateNeed
    from kirai_b200.csrc import ops

    gen = torch.Generator().manual_seed(heads * 100 + state)
    lens = [9, 64, 65, 200, 1, 33]
    offset = 7  # the state's columns start behind others
    L = offset + heads * state * vdim
    session = Session([StateNeed((L,), torch.float32)], torch.float32, page_size=4, num_pages=4, num_slots=8)
    batch = session.batch([(f"r{i}", n) for i, n in enumerate(lens)])
    T, inner = sum(lens), heads * vdim
    xbc = torch.randn((T, inner + 2 * groups * state), generator=gen)
    dt = torch.randn((T, heads + 3), generator=gen)[:, 3:]  # a run of columns of a wider tensor
    dt_bias, a_log, skip = torch.randn(heads, generator=gen), torch.randn(heads, generator=gen) * 1.5, torch.randn(heads, generator=gen)
    state0 = torch.randn((8, L), generator=gen)
    results = []
    for limits in FORMS:
        st = state0.clone().cuda()
        y = ops.ssm_walk(xbc.cuda(), dt.cuda(), dt_bias.cuda(), a_log.cuda(), skip.cuda(), st, offset, batch, heads, groups, state, vdim,
                         **limits)
        results.append((y.cpu(), st.cpu()))
    (y_c, st_c), (y_s, st_s), (y_w, st_w) = results
    assert torch.equal(st_c[:, :offset], state0[:, :offset])
    step = np.log1p(np.exp((dt + dt_bias).double().numpy()))
    starts = batch.query_start.cpu().tolist()  # (the batch orders its requests itself)
    assert sorted(b - a for a, b in zip(starts, starts[1:])) == sorted(lens)
    for r, (first, n) in enumerate(zip(starts, np.diff(starts))):
        slot = int(batch.slots[r])
        for h in range(heads):
            g = h // (heads // groups)
            rows = slice(first, first + n)
            q = xbc[rows, inner + groups * state + g * state : inner + groups * state + (g + 1) * state].double().numpy()
            k = xbc[rows, inner + g * state : inner + (g + 1) * state].double().numpy()
            v = xbc[rows, h * vdim : (h + 1) * vdim].double().numpy()
            S0 = state0[slot, offset + h * state * vdim : offset + (h + 1) * state * vdim].double().numpy().reshape(state, vdim)
            keep_log = -np.exp(float(a_log[h])) * step[rows, h]
            o, S, _, _ = _plain_scan(q, k, v, keep_log, None, step[rows, h], S0, np.zeros(state), 0.0, False)
            o = o + float(skip[h]) * v
            for name, y, st in (("chunks in a chain", y_c, st_c), ("chunks side by side", y_s, st_s), ("walk", y_w, st_w)):
                got = y[rows, h * vdim : (h + 1) * vdim].double().numpy()
                assert np.abs(got - o).max() <= 3e-5 * max(1.0, np.abs(o).max()), (name, r, h)
                got = st[slot, offset + h * state * vdim : offset + (h + 1) * state * vdim].double().numpy().reshape(state, vdim)
                assert np.abs(got - S).max() <= 3e-5 * max(1.0, np.abs(S).max()), (name, "state", r, h)


@pytest.mark.gpu
@pytest.mark.parametrize("heads,dim,vdim,cap", [(2, 8, 16, 5.0), (3, 40, 20, 15.0), (2, 128, 64, 8.0), (1, 256, 80, 2.0), (1, 3, 5, 10.0)])
def test_matrix_memory_runs_in_chunks_as_token_by_token(heads, dim, vdim, cap):
    """The same for the matrix memory, with gates that reach their cap on both sides and carried maxima on both sides
    of zero, so that within a chunk the running maximum is first the carried one and then a token's."""
    from part_helpers import Session
    from kirai_b200.parts.base import StateNeed
    from kirai_b200.csrc import ops

    gen = torch.Generator().manual_seed(heads * 100 + dim)
    lens = [9, 64, 65, 200, 1, 33]
    L = heads * (dim * vdim + dim + 1)
    session = Session([StateNeed((L,), torch.float32)], torch.float32, page_size=4, num_pages=4, num_slots=8)
    batch = session.batch([(f"r{i}", n) for i, n in enumerate(lens)])
    T = sum(lens)
    width = heads * (2 * dim + vdim + 2)
    rows_all = torch.randn((T, width + 5), generator=gen)  # further columns are left alone
    rows_all[:, width - 2 * heads : width] *= 6.0
    in_bias, keep_bias = torch.randn(heads, generator=gen), torch.randn(heads, generator=gen) + 2.0
    state0 = torch.randn((8, L), generator=gen)
    state0[:, heads * (dim * vdim + dim):] *= 4.0  # the carried maxima
    scale = dim ** -0.5
    results = []
    for limits in FORMS:
        st = state0.clone().cuda()
        o = ops.matrix_memory_walk(rows_all.cuda(), in_bias.cuda(), keep_bias.cuda(), cap, scale, st, batch, heads, dim, vdim, **limits)
        results.append((o.cpu(), st.cpu()))
    (o_c, st_c), (o_s, st_s), (o_w, st_w) = results
    R = rows_all.double().numpy()
    starts = batch.query_start.cpu().tolist()
    assert sorted(b - a for a, b in zip(starts, starts[1:])) == sorted(lens)
    for r, (first, n) in enumerate(zip(starts, np.diff(starts))):
        slot = int(batch.slots[r])
        base = state0[slot].double().numpy()
        for h in range(heads):
            rows = slice(first, first + n)
            q = R[rows, h * dim : (h + 1) * dim] * scale
            k = R[rows, heads * dim + h * dim : heads * dim + (h + 1) * dim]
            v = R[rows, 2 * heads * dim + h * vdim : 2 * heads * dim + (h + 1) * vdim]
            gi = R[rows, heads * (2 * dim + vdim) + h] + float(in_bias[h])
            gf = R[rows, heads * (2 * dim + vdim) + heads + h] + float(keep_bias[h])
            take_log = cap * np.tanh(gi / cap)
            capped = cap * np.tanh(gf / cap)
            keep_log = -np.log1p(np.exp(-capped))
            S0 = base[h * dim * vdim : (h + 1) * dim * vdim].reshape(dim, vdim)
            n0 = base[heads * dim * vdim + h * dim : heads * dim * vdim + (h + 1) * dim]
            m0 = float(base[heads * (dim * vdim + dim) + h])
            o, S, nn, m = _plain_scan(q, k, v, keep_log, take_log, None, S0, n0, m0, True)
            for name, got_o, st in (("chunks in a chain", o_c, st_c), ("chunks side by side", o_s, st_s), ("walk", o_w, st_w)):
                got = got_o[rows, h * vdim : (h + 1) * vdim].double().numpy()
                # (the read-out divides by |n . q|, a sum whose terms cancel: its 32-bit rounding shows in the quotient)
                assert np.abs(got - o).max() <= 3e-4 * max(1.0, np.abs(o).max()), (name, r, h)
                s = st[slot].double().numpy()
                for what, mine, plain_one in (("S", s[h * dim * vdim : (h + 1) * dim * vdim].reshape(dim, vdim), S),
                                              ("n", s[heads * dim * vdim + h * dim : heads * dim * vdim + (h + 1) * dim], nn),
                                              ("m", s[heads * (dim * vdim + dim) + h], m)):
                    assert np.abs(mine - plain_one).max() <= 1e-4 * max(1.0, np.abs(plain_one).max()), (name, what, r, h)


# ---- the window that keeps a sequence's first keys -------------------------------------------------------------------
ATTENTION_CASES = [  # (heads, kv heads, dim, vdim, scale, rotation, window, kept first keys), width, page size
    (attn(4, 2, 16, 16, 0.7, rot(500.0, 8, (4.0, 32, 4.0, 1.0)), 8, 3), 64, 4),
    (attn(6, 1, 12, 20, 0.9, rot(77.0, 4, (2.0, 16, 3.0, 0.5)), 5, 7), 100, 8),
    (attn(2, 2, 32, 8, 0.4, rot(10000.0, 32), 16, 0), 40, 16),
    (attn(3, 3, 10, 6, 1.1, rot(50.0, 10), 11, 1), 30, 2),
    (attn(4, 2, 64, 64, 0.125, rot(1e4, 64, (8.0, 64, 8.0, 1.0)), 33, 4), 64, 16),
    (attn(8, 2, 128, 64, 0.09, rot(1e5, 32), 40, 17), 96, 16),
    (attn(2, 1, 24, 40, 0.3, rot(300.0, 24), 1, 2), 48, 8),       # a window of the token itself, and two kept keys
    (attn(2, 1, 16, 16, 0.5, rot(300.0, 8), 64, 5), 32, 64),      # a window as wide as a page
]


def _attention_side(mixer, width):
    part, _ = _mixer(parallel(mixer, memory(1, 4, 4, 5.0)), width)
    return part.left


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mixer,width,page", ATTENTION_CASES, ids=lambda c: "x".join(str(c[k]) for k in ("heads", "kv_heads", "dim", "vdim")) if isinstance(c, dict) else str(c))
def test_windowed_attention_whole_in_portions_and_one_by_one(dtype, mixer, width, page):
    """150 tokens whole, in uneven portions, with the last ten decoded, in pairs and one by one, on a pool with no page
    to spare, so that pages the window gave back are used again; the pages of the kept first keys stay."""
    from part_helpers import Session, load_part

    part = _attention_side(mixer, width)
    w = {k: v.double() for k, v in load_part(part, dtype, seed=13).items()}
    tokens = 150
    x = (torch.randn((tokens, width), generator=torch.Generator().manual_seed(width)) * 1.5).to(dtype)
    expected = plain.windowed_attention(x.double(), w, mixer, "a.left.")
    session = Session([part.cache_need()], dtype, page_size=page, num_pages=-(-tokens // page) + 1, num_slots=2)
    for cuts in CUTS(tokens):
        close(dtype, _run_part(part, session, x, cuts), expected, f"cut as {cuts[:4]}...")
        assert all(pool.free_pages == session.cache.num_pages for pool in session.cache.tables.pools)


def _opposed_projections(part, seed, rotated):
    """Random tensors for an attention side whose query projection is minus its key projection, with nothing in the
    rotated columns of a head: a token then scores -|k|^2 against itself, whatever its place, and a token whose input
    is minus three times an earlier token's scores 3|k|^2 against that one and stands out under the softmax."""
    from kirai_b200.weights.random_init import random_tensors

    tensors = random_tensors(part.weight_specs(), seed, std=0.08, norm_jitter=0.1, dtype=torch.bfloat16)
    heads, kv_heads, dim = part.q_heads, part.kv_heads, part.head_dim
    k = tensors["a.left.k"].view(kv_heads, dim, -1).clone()
    k[:, :rotated] = 0.0
    tensors["a.left.k"] = k.reshape(kv_heads * dim, -1)
    tensors["a.left.q"] = (-k).repeat_interleave(heads // kv_heads, dim=0).reshape(heads * dim, -1)
    return tensors


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("size,keep,page", [(16, 3, 4), (21, 6, 8), (64, 1, 16), (7, 9, 4)])
def test_keys_at_the_windows_edge_and_the_kept_first_keys_stand_out(dtype, size, keep, page):
    """Pairs of (early, late) tokens of which late puts its weight on early if it sees it: early just inside the window
    (late - early = size - 1), just outside (= size; late then spreads its weight over what it does see), the last kept
    key (early = keep - 1) and the first that is not kept (early = keep) seen from far away, in a prompt and decoded.
    A window or a count of kept keys that is off by one in either direction is far outside the bound."""
    from part_helpers import Session, load_part

    mixer, width = attn(4, 2, 64, 8, 0.6, rot(100.0, 8), size, keep), 48
    part = _attention_side(mixer, width)
    w = {k: v.double() for k, v in load_part(part, dtype, tensors=_opposed_projections(part, 21, 8)).items()}
    total = 300
    x = torch.randn((total, width), generator=torch.Generator().manual_seed(size)).to(dtype)
    pairs = [(100 - (size - 1), 100), (130 - size, 130), (keep - 1, 150), (keep, 170),                 # in a prompt
             (250 - (size - 1), 250), (270 - size, 270), (keep - 1, 285), (keep, 295), (0, 299)]      # decoded
    for early, late in pairs:
        x[late] = -3.0 * x[early]
    expected = plain.windowed_attention(x.double(), w, mixer, "a.left.")
    bound = tolerance(dtype, expected.numpy())
    late_rows = [late for _, late in pairs]
    for other_size, other_keep in ((size + 1, keep), (size - 1, keep), (size, keep + 1), (size, keep - 1)):
        if other_size < 1 or other_keep < 0:
            continue
        other = plain.windowed_attention(x.double(), w, {**mixer, "mask": {"size": other_size, "keep_first": other_keep}}, "a.left.")
        assert float((other - expected)[late_rows].abs().max()) > 3 * bound, (other_size, other_keep)
    session = Session([part.cache_need()], dtype, page_size=page, num_pages=-(-total // page) + 1, num_slots=2)
    for cuts in ([total], [200] + [1] * 100, [99, 2, 30, 69] + [1] * 50 + [2] * 25):
        close(dtype, _run_part(part, session, x, cuts), expected, f"cut as {cuts[:4]}...")


# ---- two mixers side by side; batches of unequal requests -----------------------------------------------------------
SIDE_BY_SIDE_CASES = [
    (attn(4, 2, 16, 16, 0.7, rot(500.0, 8, (4.0, 32, 4.0, 1.0)), 8, 3), memory(2, 8, 16, 5.0), 64, 4),
    (attn(6, 1, 12, 20, 0.9, rot(77.0, 4, (2.0, 16, 3.0, 0.5)), 5, 7), memory(3, 10, 12, 2.0), 100, 8),
    (attn(2, 2, 32, 8, 0.4, rot(10000.0, 32), 16, 0), memory(1, 24, 20, 8.0), 40, 16),
]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", SIDE_BY_SIDE_CASES, ids=["a", "b", "c"])
def test_side_by_side_alone_and_in_batches_of_unequal_requests(dtype, case):
    """Both sides read the same rows; each output is divided by its root mean square over the width, weighted, and the
    two are averaged.  Five unequal requests, at most two at a time on two state slots and a pool that holds two
    requests' pages: portions of one beside single tokens of another, each equal to the request alone."""
    from part_helpers import Session, load_part

    left, right, width, page = case
    part, raw = _mixer(parallel(left, right), width)
    w = {k: v.double() for k, v in load_part(part, dtype, seed=width).items()}
    g = torch.Generator().manual_seed(page)
    xs = {name: (torch.randn((n, width), generator=g) * 1.5).to(dtype) for name, n in (("p", 70), ("q", 33), ("r", 9), ("s", 48), ("t", 2))}
    expected = {name: plain.parallel_mixer(x.double(), w, raw, "a.", 1e-5) for name, x in xs.items()}
    session = Session(_needs(part), dtype, page_size=page, num_pages=-(-70 // page) - (-48 // page), num_slots=2)
    alone = _run_part(part, session, xs["p"], [70])
    close(dtype, alone, expected["p"], "alone, whole")
    steps = [[("p", 40), ("q", 2)], [("p", 1), ("q", 20)], [("p", 1), ("q", 1)], [("q", 10), ("p", 28)],      # p and q end here
             [("r", 7), ("s", 1)], [("r", 1), ("s", 30)], [("s", 1), ("r", 1)], [("s", 16)],                   # r ends, then s
             [("t", 1)], [("t", 1)]]
    got = _run_together(part, session, xs, steps)
    for name in xs:
        close(dtype, got[name], expected[name], f"request {name} in batches")


# ---- experts chosen by a softmax over all of them, and a branch that every token takes ------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("count,top,ff,shared,width", [(4, 2, 24, 16, 64), (3, 1, 16, None, 40), (5, 3, 20, 28, 100), (2, 2, 12, 8, 100),
                                                       (1, 1, 8, 8, 16), (16, 4, 8, None, 24), (6, 5, 32, 40, 48)])
def test_experts_weighted_by_the_softmax_over_all(dtype, count, top, ff, shared, width):
    """The chosen experts' weights are their shares of the softmax over ALL experts (they do not sum to one unless all
    are chosen); the shared branch is added unweighted."""
    from part_helpers import DEV, load_part

    raw = {"architecture": "Figalix", "width": width, "vocab": 8, "norm": {"eps": 1e-5}, "residual_mult": 1.0,
           "layers": [layer(mamba(1, 4, 4, 1, 2, 1), moe(count, top, ff, shared))]}
    from kirai_b200.config.figalix import FigalixConfig
    from kirai_b200.models.figalix import feed_forward_for_layer
    from kirai_b200.weights.random_init import random_tensors

    cfg = FigalixConfig.from_dict(raw)
    part = feed_forward_for_layer(cfg, cfg.layers[0], "m.")
    tensors = random_tensors(part.weight_specs(), count, std=0.08, norm_jitter=0.1, dtype=torch.bfloat16)
    tensors["m.router"] = (tensors["m.router"].float() * 3.0).to(torch.bfloat16)  # shares that differ
    w = {k: v.double() for k, v in load_part(part, dtype, tensors=tensors).items()}
    x = (torch.randn((40, width), generator=torch.Generator().manual_seed(7)) * 1.5).to(dtype)
    margins = []
    expected = plain.routed_ffn(x.double(), w, raw["layers"][0]["mlp"], "m.", margins)
    sure = (margins[0] > 0.05).numpy() if dtype == torch.bfloat16 else np.ones(40, bool)
    assert sure.mean() > 0.6
    got = part.forward(x.to(DEV), None).cpu()
    assert got.dtype == torch.float32
    close(dtype, got, expected, "experts", rows=sure)
    ids, weights = plain.router_choice(x.double(), w, raw["layers"][0]["mlp"], "m.")
    if top < count:
        assert float(weights.sum(-1).min()) < 0.95  # not renormalized
    gates, chosen, mix = part.rt.ops.router_gates(x.to(DEV), part.router, top, True, over_all=True)
    for t in np.nonzero(sure)[0]:
        assert sorted(chosen[t].tolist()) == sorted(ids[t].tolist())
        want = torch.zeros(count, dtype=torch.float64)
        want[ids[t]] = weights[t]
        assert float((gates[t].cpu().double() - want).abs().max()) < 1e-5
    # one token at a time gives the same rows
    single = torch.cat([part.forward(x[i : i + 1].to(DEV), None).cpu() for i in range(12)])
    close(dtype, single, expected[:12], "one by one", rows=sure[:12])


# --------------------------------------------------------------------------- whole models (GPU)
CLOSE_CALL = 0.03  # a router margin below this may fall the other way once activations are rounded to bfloat16
SENSITIVE = 0.25   # of the bfloat16 bound: a position that moves this far when ONLY the sub-layers' inputs are rounded


class Reference(np.ndarray):
    """Plain logits [T, vocab] with ``close`` [T]: whether a token's choice of experts is a close call in some layer,
    or the plain logits themselves move by a good part of the bound when nothing but the rows that the sub-layers read
    is rounded to bfloat16 (a memory's read-out that nearly cancels before it is divided by its root mean square does
    that).  Such a token is compared in 32-bit only."""


def reference_with_close_calls(config, weights, tokens):
    margins = []
    logits = plain.forward(config, weights, tokens, margins=margins).numpy().view(Reference)
    close = (torch.stack(margins).min(dim=0).values < CLOSE_CALL).numpy() if margins else np.zeros(len(tokens), bool)
    moved = np.abs(plain.forward(config, weights, tokens, round_inputs=True).numpy() - np.asarray(logits)).max(axis=1)
    logits.close = close | (moved > SENSITIVE * tolerance("bfloat16", np.asarray(logits)))
    return logits


def check(dtype, got, reference, rows, what):
    expected = np.asarray(reference)[rows]
    assert got.shape == expected.shape, what
    diff = np.abs(got - expected).max(axis=1)
    if dtype in ("bfloat16", torch.bfloat16):
        diff = np.where(reference.close[rows], 0.0, diff)
    assert float(diff.max()) <= tolerance(dtype, reference), f"{what}: max abs diff {float(diff.max())} (bound {tolerance(dtype, reference)})"


@pytest.fixture(scope="module", params=["A", "B"])
def tiny(request, tmp_path_factory):
    raw, page, seed = TINY[request.param]
    folder = str(tmp_path_factory.mktemp(f"figalix{request.param}"))
    write_model(folder, raw, seed)
    config, weights = read_model_folder(folder)
    assert config == raw
    sequences = {rid: random_tokens(n, raw["vocab"], 300 + k)
                 for k, (rid, n) in enumerate([("a", 75), ("b", 40), ("c", 53), ("d", 9), ("e", 61), ("f", 34)])}
    reference = {rid: reference_with_close_calls(config, weights, toks) for rid, toks in sequences.items()}
    return dict(name=request.param, folder=folder, raw=raw, config=config, weights=weights, page=page,
                sequences=sequences, reference=reference)


@pytest.mark.gpu
def test_close_calls_are_few(tiny):
    for rid, reference in tiny["reference"].items():
        assert reference.close.mean() <= 0.4, rid


@pytest.mark.gpu
def test_residual_stream_after_every_layer(tiny):
    """In 32-bit the stream after each layer equals the plain one."""
    from kirai_b200.engine.batch import StepEntry
    from kirai_b200.engine.runner import ModelRunner
    from kirai_b200.parts.block import Block

    runner = ModelRunner.from_folder(tiny["folder"], dtype="float32", page_size=tiny["page"], max_tokens=128, num_slots=2)
    tokens = tiny["sequences"]["b"]
    _, streams = plain.forward(tiny["config"], tiny["weights"], tokens, return_layers=True)
    kept, original = [], Block.forward

    def recording(self, resid, *args, **kwargs):
        out = original(self, resid, *args, **kwargs)
        # a block hands on its stream and what its last sub-layer still has to add
        stream, left = out
        total = stream.double().cpu()
        if left is not None:
            rows, factor = (left.rows, left.factor) if hasattr(left, "rows") else ([left], 1.0)
            total = total + factor * sum(t.double().cpu() for t in rows)
        kept.append(total)
        return out

    Block.forward = recording
    try:
        runner.step([StepEntry(runner.cache.open("b"), tokens, [0])])
    finally:
        Block.forward = original
    assert len(kept) == len(streams)
    for index, total in enumerate(kept):
        assert float((total - streams[index]).abs().max()) < 2e-4 * max(1.0, float(streams[index].abs().max())), f"after layer {index}"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_then_last_tokens_one_by_one(tiny, dtype, tmp_path):
    from replay_client import Replay

    replay = Replay(tiny["folder"], dtype, str(tmp_path / "out"), max_tokens=160, page_size=tiny["page"])
    for rid in ("a", "d"):
        toks = tiny["sequences"][rid]
        got = replay.step([(rid, toks, range(len(toks)))], end=[rid])
        check(dtype, got, tiny["reference"][rid], list(range(len(toks))), f"whole {rid}")
    for rid in ("a", "c"):
        toks = tiny["sequences"][rid]
        head = len(toks) - 32  # every window of the tiny models passes over decoded tokens only at the end
        got = replay.step([(rid, toks[:head], [head - 1])])
        check(dtype, got, tiny["reference"][rid], [head - 1], f"{rid} prompt")
        for i in range(head, len(toks)):
            got = replay.step([(rid, [toks[i]], [0])], end=[rid] if i == len(toks) - 1 else [])
            check(dtype, got, tiny["reference"][rid], [i], f"{rid} decode at {i}")
    assert replay.close() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_prompt_of_many_chunks_whole_and_in_portions(tiny, dtype, tmp_path):
    """A prompt long enough for the recurrent mixers to take its chunks side by side, whole and beside a second request;
    the same prompt in portions that go through the chunks in a chain and through the walk; both against the plain
    model."""
    from replay_client import Replay

    toks = random_tokens(330, tiny["raw"]["vocab"], 77)
    other = tiny["sequences"]["d"]
    reference = reference_with_close_calls(tiny["config"], tiny["weights"], toks)
    rows = [0, 1, 63, 64, 65, 127, 128, 200, 255, 256, 257, 300, 328, 329]
    replay = Replay(tiny["folder"], dtype, str(tmp_path / "out"), max_tokens=512, page_size=tiny["page"])
    got = replay.step([("long", toks, rows), ("d", other, [len(other) - 1])], end=["long", "d"])
    check(dtype, got[: len(rows)], reference, rows, "whole, beside a short request")
    check(dtype, got[len(rows) :], tiny["reference"]["d"], [len(other) - 1], "the short request beside it")
    done = 0
    for size in (130, 3, 70, 1, 100, 26):  # chains of three and two chunks, walks, a single token
        want = [r - done for r in rows if done <= r < done + size]
        got = replay.step([("again", toks[done : done + size], want)], end=["again"] if done + size == len(toks) else [])
        if want:
            check(dtype, got, reference, [r + done for r in want], f"portion at {done}")
        done += size
    assert done == len(toks) and replay.close() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_down_to_two_tokens(tiny, dtype, tmp_path):
    """Portions that end inside a page, inside a window, among the kept first keys and inside the convolution's reach."""
    from replay_client import Replay

    replay = Replay(tiny["folder"], dtype, str(tmp_path / "out"), max_tokens=96, page_size=tiny["page"])
    toks = tiny["sequences"]["a"]
    for sizes in ([13, 2, 7, 16, 5, 3, 2, 11, 9, 2, 5], [2] * 37 + [1], [64, 11], [1, 1, 2, 3, 68]):
        assert sum(sizes) == len(toks)
        start = 0
        for size in sizes:
            got = replay.step([("a", toks[start : start + size], range(size))])
            check(dtype, got, tiny["reference"]["a"], list(range(start, start + size)), f"portion at {start}+{size}")
            start += size
        replay.step([], end=["a"])
    assert replay.close() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_on_a_pool_that_runs_full(tiny, dtype, tmp_path):
    """Six unequal requests, at most four live on four state slots, portions of some beside single tokens of others, on
    a pool exactly as large as the most that live requests hold at once: later requests get pages and slots that
    earlier ones gave back, and every logit equals what the request gives alone."""
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
            check(dtype, got[row : row + count], reference[rid], list(range(first, first + count)), f"mixed {rid} at {first}+{count}")
            row += count
    assert replay.close() == 0
    stats = replay.stats()
    assert stats["live_requests"] == 0
    for group in stats["groups"]:
        assert group["used"] == 0 and group["handed_out"] > group["pages"] == most // page


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(tiny, dtype, tmp_path):
    """330 tokens one by one from the first: the kept keys fill up, the windows pass over them, the states run long."""
    from replay_client import Replay

    toks = random_tokens(330, tiny["raw"]["vocab"], 17)
    reference = reference_with_close_calls(tiny["config"], tiny["weights"], toks)
    replay = Replay(tiny["folder"], dtype, str(tmp_path / "out"), max_tokens=352, page_size=tiny["page"])
    for i, token in enumerate(toks):
        got = replay.step([("long", [token], [0])])
        check(dtype, got, reference, [i], f"decode at {i}")
    assert replay.close() == 0


def test_bounds_would_show_lost_kept_keys_or_a_window_off_by_one(tiny):
    """The whole models' bound is far below what these faults cost.  (Random experts and memories add too little to a
    tiny model's logits for a fault in their weights or gates to show there: the parts' own tests compare those.)"""
    tokens, true = tiny["sequences"]["a"], np.asarray(tiny["reference"]["a"])
    bound = tolerance("bfloat16", true)

    def with_patched(name, replacement):
        original = getattr(plain, name)
        setattr(plain, name, replacement(original))
        try:
            return plain.forward(tiny["config"], tiny["weights"], tokens).numpy()
        finally:
            setattr(plain, name, original)

    no_kept = with_patched("visible_keys", lambda f: lambda T, size, keep: f(T, size, 0))
    wider = with_patched("visible_keys", lambda f: lambda T, size, keep: f(T, size + 1, keep))
    for name, other in (("kept keys", no_kept), ("window", wider)):
        assert float(np.abs(other - true).max()) > 3 * bound, name


def _margin_ok(config, weights, prompt, generated):
    logits = plain.forward(config, weights, list(prompt) + list(generated))
    top2 = torch.topk(logits[len(prompt) - 1 : -1], 2, dim=-1).values
    return bool(((top2[:, 0] - top2[:, 1]) > 2e-3).all())


def _plain_greedy(config, weights, prompt, count):
    tokens = list(prompt)
    for _ in range(count):
        logits = plain.forward(config, weights, tokens)[-1]
        tokens.append(int(torch.nonzero(logits == logits.max())[0]))
    return tokens[len(prompt):]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(tiny, dtype):
    """Five prompts through the scheduler (three at a time on three state slots, prompts in portions of 16, decode steps
    from captured graphs where the engine captures them) give the plain implementation's greedy tokens."""
    from kirai_b200 import Engine, SamplingParams

    engine = Engine(tiny["folder"], dtype=dtype, page_size=tiny["page"], max_prefill_tokens=16, max_concurrent_requests=3,
                    max_new_tokens=16, max_cache_tokens=256)
    prompts = [random_tokens(n, tiny["raw"]["vocab"], 50 + n) for n in (5, 11, 17, 3, 24)]
    outputs = engine.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=8))
    compared = 0
    for prompt, output in zip(prompts, outputs):
        expected = _plain_greedy(tiny["config"], tiny["weights"], prompt, 8)
        assert output.finish_reason == "length" and (output.prompt_tokens, output.completion_tokens) == (len(prompt), 8)
        if dtype == "float32" or _margin_ok(tiny["config"], tiny["weights"], prompt, expected):
            assert output.token_ids == expected
            compared += 1
    assert compared >= 3
    stats = engine.stats()
    assert stats["cache"]["live_requests"] == 0 and all(g["used"] == 0 for g in stats["cache"]["groups"])


@pytest.mark.gpu
def test_eviction_and_recompute_give_the_same_sampled_tokens(tiny):
    """Seeded temperature sampling on a pool too small for both requests: one is evicted, its pages and its state slots
    go back, and its recomputation (states from zero again) gives the tokens of the roomy run."""
    from kirai_b200 import Engine, SamplingParams

    params = SamplingParams(temperature=0.8, top_p=0.95, seed=5, max_new_tokens=14)
    prompts = [random_tokens(17, tiny["raw"]["vocab"], 1), random_tokens(18, tiny["raw"]["vocab"], 2)]
    roomy = Engine(tiny["folder"], dtype="float32", page_size=tiny["page"], max_new_tokens=16, max_cache_tokens=256)
    expected = [o.token_ids for o in roomy.generate(prompts, params)]
    tight = Engine(tiny["folder"], dtype="float32", page_size=tiny["page"], max_new_tokens=16, max_cache_tokens=48)
    outputs = tight.generate(prompts, params)
    assert [o.token_ids for o in outputs] == expected


@pytest.mark.gpu
def test_command_line_generates(tiny):
    prompt = random_tokens(9, tiny["raw"]["vocab"], 77)
    result = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "kirai"), "generate", "--snapshot", tiny["folder"],
                             "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "6", "--temperature", "0",
                             "--dtype", "float32", "--page-size", str(tiny["page"])], capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr
    expected = _plain_greedy(tiny["config"], tiny["weights"], prompt, 6)
    assert json.loads(result.stdout.strip().splitlines()[-1])["token_ids"] == expected
