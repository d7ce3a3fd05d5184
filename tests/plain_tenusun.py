"""A plain, slow implementation of the Tenusun decoder: whole sequences, no cache, no batching, one function per
mechanism, written out from the design's equations.  It shares no code with the library and is the oracle of the
GPU tests.

Notation.  A sequence has tokens at positions p = 0 .. n-1; ``x`` is the residual stream [n, width].  ``cfg`` is the
parsed config.json, ``w`` maps tensor names to tensors; matrices are [out, in] and applied as W x.  Everything runs
in the dtype of the weights handed in (the tests use float64).
"""
from __future__ import annotations

import math

import torch


# ------------------------------------------------------------------ small pieces

def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def layer_norm(x, weight, bias, eps):
    """(x - mean) / sqrt(var + eps) * weight + bias over the last axis, var the mean of the squared deviations."""
    mu = x.mean(-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * weight + bias


def sigmoid(z):
    return 1 / (1 + torch.exp(-z))


def lin(w, h):
    return h @ w.T


# ------------------------------------------------------------------ rotation

def plain_frequencies(dims, base):
    """f_i = base^(-2i/dims), i < dims/2."""
    return [base ** (-2.0 * i / dims) for i in range(dims // 2)]


def stretched_frequencies(dims, base, scaling):
    """The frequencies and the factor on cos and sin where a ``scaling`` object (factor, original, fast, slow) is given:
    entries that turn fast keep their frequency, those that turn slowly have it divided by ``factor``, a ramp in between."""
    f = plain_frequencies(dims, base)
    if scaling is None:
        return f, 1.0
    factor, original = scaling["factor"], scaling["original"]

    def where(turns):
        return dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(base))
    lo = max(math.floor(where(scaling["fast"])), 0)
    hi = min(math.ceil(where(scaling["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_half(u, dims, freqs, magnitude=1.0, first=0):
    """u [n, ..., D]: entry i < dims/2 pairs with entry i + dims/2; the pair (a, b) of the token at position p becomes
    (a cos - b sin, b cos + a sin) with the angle p * freqs[i], cos and sin multiplied by ``magnitude``.  Entries from
    ``dims`` on stay.  ``first``: the position of the first row."""
    out = u.clone()
    n = u.shape[0]
    pos = torch.arange(first, first + n, dtype=u.dtype)
    shape = [n] + [1] * (u.dim() - 2)
    half = dims // 2
    for i in range(half):
        a = pos * freqs[i]
        c, s = (torch.cos(a) * magnitude).view(shape), (torch.sin(a) * magnitude).view(shape)
        lo, hi = u[..., i], u[..., i + half]
        out[..., i] = lo * c - hi * s
        out[..., i + half] = hi * c + lo * s
    return out


# ------------------------------------------------------------------ masks and softmax

def causal_mask(n, size=None):
    """[n, n] bool: query i sees key j iff 0 <= i - j (< size, where a size is given)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    seen = j <= i
    if size is not None:
        seen = seen & (i - j < size)
    return seen


def softmax_rows(s, visible, extra_one=False):
    """Softmax of every row of s over the visible places; ``extra_one``: one more place of score 0 joins the denominator
    and carries nothing: p_j = exp(s_j) / (1 + sum exp(s_j))."""
    s = torch.where(visible, s, torch.full_like(s, -math.inf))
    m = s.max(-1, keepdim=True).values
    if extra_one:
        m = torch.clamp(m, min=0.0)
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if extra_one:
        den = den + torch.exp(-m)
    return e / den


# ------------------------------------------------------------------ latent attention

def latent_attention_mixer(h, m, w, p, eps):
    """Queries through a low-rank row, keys and values from another one; a rotated key part shared by the heads;
    a sliding window; ordinary softmax."""
    n = h.shape[0]
    H, D, R, Dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms_unit(lin(w[p + "dq"], h), eps) * w[p + "dq.norm"]
    q = lin(w[p + "uq"], cq).view(n, H, D + R)
    down = lin(w[p + "dkv"], h)
    c = rms_unit(down[:, :rank], eps) * w[p + "dkv.norm"]
    freqs = plain_frequencies(R, m["rot"]["base"])
    k_rot = rotate_half(down[:, rank:], R, freqs)                              # [n, R], one for all heads
    q_rot = rotate_half(q[..., D:], R, freqs)                                  # [n, H, R]
    k_plain = lin(w[p + "uk"], c).view(n, H, D)
    v = lin(w[p + "uv"], c).view(n, H, Dv)
    seen = causal_mask(n, (m.get("mask") or {}).get("size"))
    heads = []
    for a in range(H):
        s = (q[:, a, :D] @ k_plain[:, a].T + q_rot[:, a] @ k_rot.T) * m["scale"]
        heads.append(softmax_rows(s, seen) @ v[:, a])
    return lin(w[p + "o"], torch.stack(heads, dim=1).reshape(n, H * Dv))


# ------------------------------------------------------------------ grouped attention with a sink, value mixing and an output gate

def attention_values(h, m, w, p, v_first):
    """The values a layer keeps: its own, or, in every value-mixing layer after the first such, a blend with the first one's."""
    n = h.shape[0]
    v = lin(w[p + "v"], h).view(n, m["kv_heads"], m["vdim"])
    if m.get("v_mix") and v_first is not None:
        lam = w[p + "vmix"]
        v = (1 - lam) * v + lam * v_first
    return v


def attention_mixer(h, m, w, p, v):
    n = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m["rot"]
    freqs, mag = stretched_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    q = rotate_half(lin(w[p + "q"], h).view(n, H, D), rot["dims"], freqs, mag)
    k = rotate_half(lin(w[p + "k"], h).view(n, G, D), rot["dims"], freqs, mag)
    seen = causal_mask(n)
    heads = []
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * m["scale"]
        heads.append(softmax_rows(s, seen, extra_one=True) @ v[:, g])
    o = torch.stack(heads, dim=1).reshape(n, H * Dv) * sigmoid(lin(w[p + "g"], h))
    return lin(w[p + "o"], o)


# ------------------------------------------------------------------ feed-forwards

def dense_ff(h, mlp, w, p):
    """g = min(gate, limit), u = clamp(up, -limit, limit); down(g sigmoid(1.702 g) (u + 1))."""
    lim = mlp["limit"]
    g = torch.clamp(lin(w[p + "gate"], h), max=lim)
    u = torch.clamp(lin(w[p + "up"], h), min=-lim, max=lim)
    return lin(w[p + "down"], g * sigmoid(1.702 * g) * (u + 1))


ROUTER_GAPS = None      # a list: every call of ``route`` appends, a token, by how little its choice was made (for the tests)


def route(h, mlp, w, p):
    """[(expert, weight)] a token.  Scores are sigmoids of the router's logits; the choice reads score + correction, first among
    groups of neighbouring experts (a group counts the sum of its two largest; only the best ``keep`` groups stay), then the
    ``top`` largest among what stays; the weights are the plain scores of the chosen."""
    r = mlp["router"]
    E, top = r["experts"], r["top"]
    s = sigmoid(lin(w[p + "router"].to(h.dtype), h))
    choice = s + w[p + "correction"].to(h.dtype)
    groups = r.get("groups")
    out, gaps = [], []
    for t in range(h.shape[0]):
        c = choice[t].clone()
        gap = math.inf
        if groups is not None and groups["count"] > 1:
            per = E // groups["count"]
            totals = []
            for g in range(groups["count"]):
                best = torch.sort(c[g * per:(g + 1) * per], descending=True).values
                totals.append(float(best[:2].sum()))
            order = sorted(range(groups["count"]), key=lambda g: (-totals[g], g))
            if groups["keep"] < groups["count"]:
                gap = totals[order[groups["keep"] - 1]] - totals[order[groups["keep"]]]
            for g in order[groups["keep"]:]:
                c[g * per:(g + 1) * per] = -math.inf
        ranked = sorted(range(E), key=lambda e: (-float(c[e]), e))
        if top < E and c[ranked[top]] > -math.inf:
            gap = min(gap, float(c[ranked[top - 1]] - c[ranked[top]]))
        gaps.append(gap)
        out.append([(e, s[t, e]) for e in ranked[:top]])
    if ROUTER_GAPS is not None:
        ROUTER_GAPS.append(torch.tensor(gaps))
    return out


def expert(h, w, p):
    z = lin(w[p + "gate"], h)
    return lin(w[p + "down"], z * sigmoid(z) * lin(w[p + "up"], h))


def moe_ff(h, mlp, w, p):
    rows = []
    for t, chosen in enumerate(route(h, mlp, w, p)):
        rows.append(sum(weight * expert(h[t], w, f"{p}e{e}.") for e, weight in chosen))
    return torch.stack(rows)


# ------------------------------------------------------------------ the model

def hidden_states(cfg, w, tokens, keep_layers=False):
    """The residual stream after the last layer [n, width] (``keep_layers``: the list of streams after every layer too)."""
    eps = cfg["norm"]["eps"]
    x = torch.stack([w["embed"][t] for t in tokens]) * cfg["embedding"]["scale"]
    v_first, after = None, []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        if layer["type"] == "latent_attention":
            y = latent_attention_mixer(h, m, w, p + "mix.", eps)
        elif layer["type"] == "attention":
            v = attention_values(h, m, w, p + "mix.", v_first)
            if m.get("v_mix") and v_first is None:
                v_first = v
            y = attention_mixer(h, m, w, p + "mix.", v)
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        x = x + layer_norm(y, w[p + "norm1b"], w[p + "norm1b.b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps)
            y = dense_ff(h, mlp, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(h, mlp, w, p + "mlp.")
            x = x + layer_norm(y, w[p + "norm2b"], w[p + "norm2b.b"], eps)
        after.append(x)
    return (x, after) if keep_layers else x


def logits(cfg, w, tokens):
    """[n, vocab]: the final norm, then the embedding table itself (without its scale) as the head."""
    x = hidden_states(cfg, w, tokens)
    return lin(w["embed"], layer_norm(x, w["final.norm"], w["final.norm.b"], cfg["norm"]["eps"]))


def greedy(cfg, w, prompt, n_new):
    tokens, out = list(prompt), []
    for _ in range(n_new):
        t = int(torch.argmax(logits(cfg, w, tokens)[-1]))
        out.append(t)
        tokens.append(t)
    return out
