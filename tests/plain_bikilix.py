"""A plain, slow implementation of the Bikilix decoder: whole sequences, no cache, one function per mechanism,
64-bit arithmetic on the CPU.  It shares no code with the framework; model folders are read with the plain reader
of ``plain_qwen3``.

Notation: T tokens, E the model width, x the residual stream [T, E], n the normed rows a sub-layer reads, x0 the
embedding's rows.
"""
import math

import torch

F = torch.float64


def unit_norm(x, w, eps, centre=0.0):
    """x / sqrt(mean(x^2) + eps) * (centre + w) over the last axis: ``centre`` 1 when the tensor holds the weight minus one."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * (centre + w)


def relu_squared(z):
    return torch.clamp(z, min=0.0) ** 2


def pair_frequencies(rot):
    """One frequency per pair of columns: f_i = base^(-2i/dims); with ``scaling`` the frequencies from index ``lo`` to
    ``hi`` slide from f_i to f_i / factor.  Returns (frequencies, the factor on cosine and sine)."""
    dims, base = rot["dims"], rot["base"]
    freq = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(freq, dtype=F), 1.0

    def index_of(turns):
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(sc["fast"])), 0)
    hi = min(math.ceil(index_of(sc["slow"])), dims - 1)
    out = []
    for i, f in enumerate(freq):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / sc["factor"] * ramp + f * (1.0 - ramp))
    return torch.tensor(out, dtype=F), 0.1 * math.log(sc["factor"]) + 1.0


def rotate_neighbours(x, positions, rot, first=0):
    """Rotates columns [first, first + dims) of x [T, heads, d]: column first + 2i with its neighbour first + 2i + 1 by
    the angle position * f_i."""
    dims = rot["dims"]
    freq, amplitude = pair_frequencies(rot)
    # the angle is a 32-bit product of a 32-bit position and a 32-bit frequency in the design
    angle = (positions.to(torch.float32)[:, None] * freq.to(torch.float32)[None, :]).to(F)
    cos, sin = angle.cos()[:, None, :] * amplitude, angle.sin()[:, None, :] * amplitude
    u, v = x[..., first : first + dims : 2], x[..., first + 1 : first + dims : 2]
    y = x.clone()
    y[..., first : first + dims : 2] = u * cos - v * sin
    y[..., first + 1 : first + dims : 2] = v * cos + u * sin
    return y


def softmax_rows(scores, visible):
    return torch.softmax(scores.masked_fill(~visible, float("-inf")), dim=-1)


def window_attention(n, w, m, prefix, probabilities=None):
    """Grouped-query attention with biases on q, k, v, a rotated leading part of every head and a sliding window
    (position i sees j when 0 <= i - j < size)."""
    T = n.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = torch.arange(T)
    q = (n @ w[prefix + "q"].T + w[prefix + "q.b"]).view(T, H, d)
    k = (n @ w[prefix + "k"].T + w[prefix + "k.b"]).view(T, G, d)
    v = (n @ w[prefix + "v"].T + w[prefix + "v.b"]).view(T, G, dv)
    q, k = rotate_neighbours(q, positions, m["rot"]), rotate_neighbours(k, positions, m["rot"])
    i, j = positions[:, None], positions[None, :]
    visible = j <= i
    if m.get("mask"):
        visible = visible & (i - j < m["mask"]["size"])
    per = H // G
    heads = []
    for h in range(H):
        p = softmax_rows((q[:, h] @ k[:, h // per].T) * m["scale"], visible)
        if probabilities is not None:
            probabilities.append(p)
        heads.append(p @ v[:, h // per])
    return torch.cat(heads, dim=1) @ w[prefix + "o"].T


def latent_attention(n, w, m, prefix, eps, probabilities=None):
    """Queries through a normed latent; keys and values of all heads from one normed latent a token, plus one rotated
    key part that the heads share; causal; the heads' outputs gated by sigmoid(W_g n)."""
    T = n.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = torch.arange(T)
    q = (unit_norm(n @ w[prefix + "dq"].T, w[prefix + "dq.norm"], eps) @ w[prefix + "uq"].T).view(T, H, d + r)
    q = rotate_neighbours(q, positions, m["rot"], first=d)
    down = n @ w[prefix + "dkv"].T
    latent = unit_norm(down[:, :rank], w[prefix + "dkv.norm"], eps)
    shared = rotate_neighbours(down[:, rank:].reshape(T, 1, r), positions, m["rot"])[:, 0]
    keys = (latent @ w[prefix + "uk"].T).view(T, H, d)
    values = (latent @ w[prefix + "uv"].T).view(T, H, dv)
    visible = positions[None, :] <= positions[:, None]
    heads = []
    for h in range(H):
        p = softmax_rows((q[:, h, :d] @ keys[:, h].T + q[:, h, d:] @ shared.T) * m["scale"], visible)
        if probabilities is not None:
            probabilities.append(p)
        heads.append(p @ values[:, h])
    return (torch.cat(heads, dim=1) * torch.sigmoid(n @ w[prefix + "g"].T)) @ w[prefix + "o"].T


def dense_ffn(n, w, prefix):
    return relu_squared(n @ w[prefix + "up"].T) @ w[prefix + "down"].T


def expert(n, w, prefix, limit):
    g = torch.clamp(n @ w[prefix + "gate"].T, max=limit)
    u = torch.clamp(n @ w[prefix + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[prefix + "down"].T


def router_choice(n, w, mlp, prefix, margins=None):
    """(chosen experts [T, top], their weights [T, top]).  Scores are sigmoid of the 32-bit logits; the choice looks at
    score + correction, only inside the ``keep`` groups whose two largest such numbers sum highest; the weights are the
    scores themselves.  ``margins`` collects, per token, the smallest gap that decided a choice."""
    router = mlp["router"]
    E, top = router["experts"], router["top"]
    groups, keep = (router["groups"]["count"], router["groups"]["keep"]) if router.get("groups") else (1, 1)
    score = torch.sigmoid(n @ w[prefix + "router"].T)
    choice = score + w[prefix + "correction"]
    T = n.shape[0]
    size = E // groups
    grouped = choice.view(T, groups, size)
    group_score = grouped.topk(min(2, size), dim=-1).values.sum(-1)
    ranked = group_score.sort(dim=-1, descending=True)
    kept = torch.zeros(T, groups, dtype=torch.bool)
    kept.scatter_(1, ranked.indices[:, :keep], True)
    open_choice = choice.masked_fill(~kept[:, :, None].expand(T, groups, size).reshape(T, E), float("-inf"))
    ordered = open_choice.sort(dim=-1, descending=True)
    ids = ordered.indices[:, :top]
    if margins is not None:
        gap = torch.full((T,), float("inf"), dtype=F)
        if keep < groups:
            gap = torch.minimum(gap, ranked.values[:, keep - 1] - ranked.values[:, keep])
        if top < ordered.values.shape[1]:
            gap = torch.minimum(gap, (ordered.values[:, top - 1] - ordered.values[:, top]).nan_to_num(posinf=float("inf")))
        margins.append(gap)
    return ids, score.gather(1, ids)


def routed_ffn(n, w, mlp, prefix, margins=None):
    ids, weights = router_choice(n, w, mlp, prefix, margins)
    out = torch.zeros(n.shape[0], w[prefix + "e0.down"].shape[0], dtype=F)
    for e in range(mlp["router"]["experts"]):
        rows, slot = (ids == e).nonzero(as_tuple=True)
        if rows.numel():
            out[rows] += weights[rows, slot][:, None] * expert(n[rows], w, f"{prefix}e{e}.", mlp["expert"]["limit"])
    return out


def passes(config):
    """The runs of layers: a list of (pass number or None, [layer indices]); a looped stretch is one entry a pass."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(None, list(range(count)))]
    start, stop = loop.get("start", 0), loop["stop"]
    out = [(None, list(range(start)))] if start else []
    out += [(t, list(range(start, stop))) for t in range(loop["times"])]
    if stop < count:
        out.append((None, list(range(stop, count))))
    return out


def forward(config, weights, tokens, keep_layers=False, margins=None):
    """Logits [T, vocab] (float32) of a whole sequence; with ``keep_layers`` also the stream after every layer run."""
    w = {name: t.to(F) for name, t in weights.items()}
    eps = config["norm"]["eps"]
    x0 = w["embed"][torch.as_tensor(list(tokens), dtype=torch.long)] * config["embedding"]["scale"]
    x = x0
    kept = []
    for number, indices in passes(config):
        if number is not None:
            x = torch.cat([x, x0], dim=1) @ w["loop.in"].T + w["loop.step"][number]
        for index in indices:
            layer, base = config["layers"][index], f"l{index}."
            n = unit_norm(x, w[base + "norm1"], eps, 1.0)
            if layer["type"] == "attention":
                a = window_attention(n, w, layer["mixer"], base + "mix.")
            else:
                a = latent_attention(n, w, layer["mixer"], base + "mix.", eps)
            x = x + unit_norm(a, w[base + "norm1b"], eps, 1.0)
            mlp = layer["mlp"]
            if mlp is not None:
                n = unit_norm(x, w[base + "norm2"], eps, 1.0)
                f = dense_ffn(n, w, base + "mlp.") if mlp["kind"] == "dense" else routed_ffn(n, w, mlp, base + "mlp.", margins)
                x = x + unit_norm(f, w[base + "norm2b"], eps, 1.0)
            kept.append(x.to(torch.float32))
    logits = (unit_norm(x, w["final.norm"], eps, 1.0) @ w["embed"].T).to(torch.float32)
    return (logits, torch.stack(kept)) if keep_layers else logits
