"""A plain, slow implementation of the Figalix decoder: whole sequences, no cache, one function per mechanism,
64-bit arithmetic on the CPU.  It shares no code with the framework; model folders are read with the plain reader
of ``plain_qwen3``.

Notation: T tokens, E the model width, x the residual stream [T, E], n the normed rows a sub-layer reads, c the
configuration as the dict that config.json holds, w a dict of tensors by name.
"""
import math

import torch

F = torch.float64


# ---- norms and activations --------------------------------------------------------------------------------------
def dynamic_tanh(x, w, prefix):
    """tanh(alpha x) * weight + bias: no statistics of the row at all."""
    return torch.tanh(w[prefix + ".alpha"] * x) * w[prefix] + w[prefix + ".b"]


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def log_sigmoid(z):
    return -softplus(-z)


# ---- rotation ---------------------------------------------------------------------------------------------------
def stretched_frequencies(rot):
    """(f [dims/2], amplitude): f_i = base^(-2i/dims); with ``scaling`` the frequencies whose index lies above a ramp
    between two wavelengths are divided by ``factor`` (blended inside the ramp), and cos and sin grow by
    0.1 ln(factor) + 1."""
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=F), 1.0

    def index_of(turns):
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(sc["fast"])), 0)
    hi = min(math.ceil(index_of(sc["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
        out.append(fi / sc["factor"] * ramp + fi * (1.0 - ramp))
    return torch.tensor(out, dtype=F), 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x, positions, rot):
    """The first ``dims`` columns of every head of x [T, heads, d]: column i with column i + dims/2."""
    dims = rot["dims"]
    half = dims // 2
    freq, amplitude = stretched_frequencies(rot)
    # the design multiplies a 32-bit position by a 32-bit frequency
    angle = (positions.to(torch.float32)[:, None] * freq.to(torch.float32)[None, :]).to(F)
    cos, sin = angle.cos()[:, None, :] * amplitude, angle.sin()[:, None, :] * amplitude
    u, v = x[..., :half], x[..., half:dims]
    y = x.clone()
    y[..., :half] = u * cos - v * sin
    y[..., half:dims] = v * cos + u * sin
    return y


# ---- the left mixer: attention under a window that keeps a sequence's first tokens ------------------------------------
def visible_keys(T, size, keep_first):
    """[T, T] bool: row i sees column j when j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def windowed_attention(n, w, m, prefix):
    T = n.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = torch.arange(T)
    q = rotate((n @ w[prefix + "q"].T).view(T, H, d), positions, m["rot"])
    k = rotate((n @ w[prefix + "k"].T).view(T, G, d), positions, m["rot"])
    v = (n @ w[prefix + "v"].T).view(T, G, dv)
    gate = torch.sigmoid(n @ w[prefix + "g"].T)  # [T, H]: one number a head
    see = visible_keys(T, m["mask"]["size"], m["mask"]["keep_first"])
    heads = []
    for h in range(H):
        g = h // (H // G)
        scores = (q[:, h] @ k[:, g].T) * m["scale"]
        p = torch.softmax(scores.masked_fill(~see, float("-inf")), dim=-1)
        heads.append((p @ v[:, g]) * gate[:, h : h + 1])
    return torch.cat(heads, dim=-1) @ w[prefix + "o"].T


# ---- the right mixer: a matrix memory with exponential gates --------------------------------------------------------------
def matrix_memory(n, w, m, prefix, eps):
    T = n.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (n @ w[prefix + "q"].T).view(T, H, d) * d ** -0.5
    k = (n @ w[prefix + "k"].T).view(T, H, d)
    v = (n @ w[prefix + "v"].T).view(T, H, dv)
    log_in = cap * torch.tanh((n @ w[prefix + "i"].T + w[prefix + "i.b"]) / cap)          # [T, H]
    log_keep = log_sigmoid(cap * torch.tanh((n @ w[prefix + "f"].T + w[prefix + "f.b"]) / cap))
    S = torch.zeros(H, d, dv, dtype=F)
    norm = torch.zeros(H, d, dtype=F)
    peak = torch.zeros(H, dtype=F)  # the running maximum starts at 0
    rows = []
    for t in range(T):
        new_peak = torch.maximum(log_keep[t] + peak, log_in[t])
        keep = torch.exp(log_keep[t] + peak - new_peak)
        take = torch.exp(log_in[t] - new_peak)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        norm = keep[:, None] * norm + take[:, None] * k[t]
        peak = new_peak
        top = torch.einsum("hdv,hd->hv", S, q[t])
        bottom = torch.maximum((norm * q[t]).sum(-1).abs(), torch.exp(-peak)) + 1e-6
        rows.append(unit_rms(top / bottom[:, None], eps).reshape(-1))
    o = torch.stack(rows) * w[prefix + "norm"] * torch.sigmoid(n @ w[prefix + "g"].T)
    return o @ w[prefix + "o"].T


def parallel_mixer(n, w, m, prefix, eps):
    left = windowed_attention(n, w, m["left"], prefix + "left.")
    right = matrix_memory(n, w, m["right"], prefix + "right.", eps)
    return 0.5 * (unit_rms(left, eps) * w[prefix + "left.out"] + unit_rms(right, eps) * w[prefix + "right.out"])


# ---- the state-space mixer ----------------------------------------------------------------------------------------------
def causal_convolution(x, taps_w, bias):
    """x [T, C]; taps_w [C, K], whose last column weighs the current token; zeros before the start."""
    T, C = x.shape
    K = taps_w.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=x.dtype), x], dim=0)
    out = bias.expand(T, C).clone()
    for j in range(K):
        out = out + padded[j : j + T] * taps_w[:, j]
    return out


def state_space(n, w, m, prefix, eps):
    T = n.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = n @ w[prefix + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner : 2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N :]
    xbc = silu(causal_convolution(xbc, w[prefix + "conv"], w[prefix + "conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner : inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N :].view(T, G, N)
    dt = softplus(dt + w[prefix + "dt_bias"])                       # [T, H]
    decay = torch.exp(-torch.exp(w[prefix + "A_log"]) * dt)         # [T, H]
    S = torch.zeros(H, N, P, dtype=F)
    rows = []
    for t in range(T):
        y = []
        for h in range(H):
            g = h // (H // G)
            S[h] = decay[t, h] * S[h] + dt[t, h] * B[t, g][:, None] * x[t, h][None, :]
            y.append(S[h].T @ C[t, g] + w[prefix + "D"][h] * x[t, h])
        rows.append(torch.cat(y))
    y = torch.stack(rows) * silu(z)
    parts = m["norm_groups"]
    y = unit_rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[prefix + "norm"]
    return y @ w[prefix + "o"].T


# ---- feed-forwards ------------------------------------------------------------------------------------------------------
def gated_ffn(n, w, prefix):
    return (silu(n @ w[prefix + "gate"].T) * (n @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def router_choice(n, w, mlp, prefix, margins=None):
    """(chosen ids [T, top], their weights [T, top]): the largest of softmax over ALL experts, weights as they are.
    ``margins`` (a list) receives [T]: how far the last chosen logit lies above the first one left out."""
    logits = n @ w[prefix + "router"].T
    top = mlp["router"]["top"]
    weights, ids = torch.topk(torch.softmax(logits, dim=-1), top, dim=-1)
    if margins is not None:
        ranked = logits.sort(dim=-1, descending=True).values
        margins.append(ranked[:, top - 1] - ranked[:, top] if top < logits.shape[1] else torch.full((n.shape[0],), math.inf, dtype=F))
    return ids, weights


def routed_ffn(n, w, mlp, prefix, margins=None):
    ids, weights = router_choice(n, w, mlp, prefix, margins)
    out = torch.zeros(n.shape[0], w[prefix + "e0.down"].shape[0], dtype=F)
    for t in range(n.shape[0]):
        for e, g in zip(ids[t].tolist(), weights[t]):
            out[t] += g * gated_ffn(n[t : t + 1], w, f"{prefix}e{e}.")[0]
    if mlp.get("shared") is not None:
        out = out + gated_ffn(n, w, prefix + "shared.")
    return out


# ---- the model ----------------------------------------------------------------------------------------------------------
def forward(c, w, tokens, return_layers=False, margins=None, round_inputs=False):
    """Logits [T, vocab] of a whole sequence (and the stream after every layer).  ``margins`` (a list) receives one
    [T] tensor per layer with routed experts, see ``router_choice``.  ``round_inputs`` rounds the rows that every
    sub-layer reads to bfloat16 and nothing else: how far the logits move then says which positions are sensitive to
    rounding at all."""
    w = {name: (t.to(F) if t.is_floating_point() else t) for name, t in w.items()}
    eps, mult = c["norm"]["eps"], c["residual_mult"]
    x = w["embed"][torch.tensor(tokens)]
    streams = []
    for i, layer in enumerate(c["layers"]):
        base = f"l{i}."
        n = dynamic_tanh(x, w, base + "norm1")
        if round_inputs:
            n = n.to(torch.bfloat16).to(F)
        if layer["type"] == "parallel":
            x = x + mult * parallel_mixer(n, w, layer["mixer"], base + "mix.", eps)
        elif layer["type"] == "mamba2":
            x = x + mult * state_space(n, w, layer["mixer"], base + "mix.", eps)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp is not None:
            n = dynamic_tanh(x, w, base + "norm2")
            if round_inputs:
                n = n.to(torch.bfloat16).to(F)
            if mlp["kind"] == "dense":
                x = x + mult * gated_ffn(n, w, base + "mlp.")
            else:
                x = x + mult * routed_ffn(n, w, mlp, base + "mlp.", margins)
        streams.append(x)
    logits = dynamic_tanh(x, w, "final.norm") @ w["embed"].T
    cap = c.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(streams)) if return_layers else logits
