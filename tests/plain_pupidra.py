"""A plain, slow implementation of the Pupidra decoder: whole sequences, no cache, no batching, one function per
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


def sigmoid(z):
    return 1 / (1 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def relu2(z):
    return torch.clamp(z, min=0) ** 2


def lin(w, h, b=None):
    y = h @ w.T
    return y if b is None else y + b


def softmax_rows(s, visible):
    """Softmax of every row of s over the places where ``visible`` is true (every row sees at least one place)."""
    s = torch.where(visible, s, torch.full_like(s, -math.inf))
    e = torch.exp(s - s.max(-1, keepdim=True).values)
    return e / e.sum(-1, keepdim=True)


# ------------------------------------------------------------------ embedding

def embed(tokens, w, big):
    """Token rows plus bigram rows: (previous * mul_prev + current * mul_cur) mod buckets, and row ``buckets`` for the
    first token of a sequence (``big`` None: token rows alone)."""
    if big is None:
        return torch.stack([w["embed"][t] for t in tokens])
    rows = []
    for p, t in enumerate(tokens):
        r = big["buckets"] if p == 0 else (tokens[p - 1] * big["mul_prev"] + t * big["mul_cur"]) % big["buckets"]
        rows.append(w["embed"][t] + w["bigram"][r])
    return torch.stack(rows)


# ------------------------------------------------------------------ softmax attention with a distance bias

def distance_slopes(heads):
    return [2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)]


def window_keep_mask(n, size, keep_first):
    """[n, n] bool: query i sees key j iff j <= i and (i - j < size or j < keep_first); size None: every j <= i."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    seen = j <= i
    if size is not None:
        seen = seen & ((i - j < size) | (j < keep_first))
    return seen


def biased_attention(q, k, v, scale, size, keep_first):
    """q [n, H, D], k [n, G, D], v [n, G, Dv] -> [n, H, Dv].  score(i, j) = q_i . k_j * scale - slope_h (i - j)."""
    n, H, _ = q.shape
    G = k.shape[1]
    seen = window_keep_mask(n, size, keep_first)
    dist = (torch.arange(n)[:, None] - torch.arange(n)[None, :]).to(q.dtype)
    out = []
    for h, slope in enumerate(distance_slopes(H)):
        c = h // (H // G)
        s = (q[:, h] @ k[:, c].T) * scale - slope * dist
        out.append(softmax_rows(s, seen) @ v[:, c])
    return torch.stack(out, dim=1)


def attention_keys_values(h, m, w, p, eps):
    """Keys (unit-normed head by head) and values of an attention mixer that has projections of its own."""
    n = h.shape[0]
    k = rms_unit(lin(w[p + "k"], h, w[p + "k.b"]).view(n, m["kv_heads"], m["dim"]), eps)
    v = lin(w[p + "v"], h, w[p + "v.b"]).view(n, m["kv_heads"], m["vdim"])
    return k, v


def attention_mixer(h, m, w, p, eps, keys_values):
    n = h.shape[0]
    q = rms_unit(lin(w[p + "q"], h, w[p + "q.b"]).view(n, m["heads"], m["dim"]), eps)
    k, v = keys_values
    mask = m.get("mask")
    o = biased_attention(q, k, v, m["scale"], None if mask is None else mask["size"], 0 if mask is None else mask.get("keep_first", 0))
    return lin(w[p + "o"], o.reshape(n, -1), w[p + "o.b"])


# ------------------------------------------------------------------ latent attention

def rotate_pairs(u, dims, base):
    """u [n, ..., D]: neighbours (2i, 2i+1) of the first ``dims`` entries are turned by the angle p * base^(-2i/dims)."""
    out = u.clone()
    n = u.shape[0]
    pos = torch.arange(n, dtype=u.dtype)
    for i in range(dims // 2):
        a = pos * (base ** (-2.0 * i / dims))
        c, s = torch.cos(a), torch.sin(a)
        while c.dim() < u.dim() - 1:
            c, s = c[:, None], s[:, None]
        a0, a1 = u[..., 2 * i], u[..., 2 * i + 1]
        out[..., 2 * i] = a0 * c - a1 * s
        out[..., 2 * i + 1] = a1 * c + a0 * s
    return out


def latent_attention_mixer(h, m, w, p, eps):
    n = h.shape[0]
    H, D, R, Dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = lin(w[p + "q"], h).view(n, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_pairs(q[..., D:], m["rot"]["dims"], m["rot"]["base"])
    down = lin(w[p + "dkv"], h)
    c = rms_unit(down[:, :rank], eps) * w[p + "dkv.norm"]
    k_rot = rotate_pairs(down[:, rank:], m["rot"]["dims"], m["rot"]["base"])
    k_plain = lin(w[p + "uk"], c).view(n, H, D)
    v = lin(w[p + "uv"], c).view(n, H, Dv)
    gate = sigmoid(lin(w[p + "g"], h))                       # [n, H]
    seen = window_keep_mask(n, None, 0)
    out = []
    for hd in range(H):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ k_rot.T) * m["scale"]
        out.append((softmax_rows(s, seen) @ v[:, hd]) * gate[:, hd: hd + 1])
    return lin(w[p + "o"], torch.stack(out, dim=1).reshape(n, -1))


# ------------------------------------------------------------------ the state-space mixer

def causal_conv(u, taps_w, bias):
    """u [n, C]; y_t = bias + sum_j taps_w[:, j] * u_(t - taps + 1 + j), zeros before the start."""
    n, _ = u.shape
    taps = taps_w.shape[1]
    y = torch.zeros_like(u) + bias
    for j in range(taps):
        shift = taps - 1 - j
        if shift < n:
            y[shift:] += u[: n - shift] * taps_w[:, j]
    return y


def ssm_recurrence(xs, B, C, dt, A, D):
    """xs [n, H, P], B, C [n, G, N], dt [n, H], A [H] (negative), D [H] -> y [n, H, P].
    S_t = exp(A dt) S_(t-1) + dt B_t x_t^T, y_t = S_t^T C_t + D x_t."""
    n, H, P = xs.shape
    G, N = B.shape[1], B.shape[2]
    y = torch.zeros_like(xs)
    for h in range(H):
        g = h // (H // G)
        S = torch.zeros(N, P, dtype=xs.dtype)
        for t in range(n):
            S = torch.exp(A[h] * dt[t, h]) * S + dt[t, h] * torch.outer(B[t, g], xs[t, h])
            y[t, h] = S.T @ C[t, g] + D[h] * xs[t, h]
    return y


def mamba2_mixer(h, m, w, p, eps):
    n = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = lin(w[p + "in"], h)
    z, xbc, dt = proj[:, :inner], proj[:, inner: 2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    xs = xbc[:, :inner].reshape(n, H, P)
    B = xbc[:, inner: inner + G * N].reshape(n, G, N)
    C = xbc[:, inner + G * N:].reshape(n, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    y = ssm_recurrence(xs, B, C, dt, -torch.exp(w[p + "A_log"]), w[p + "D"]).reshape(n, inner)
    y = y * silu(z)
    parts = m["norm_groups"]
    y = rms_unit(y.view(n, parts, inner // parts), eps).reshape(n, inner) * w[p + "norm"]
    return lin(w[p + "o"], y)


# ------------------------------------------------------------------ feed-forward

def expert(h, w, p):
    return lin(w[p + "down"], relu2(lin(w[p + "up"], h)))


ROUTER_GAPS = None      # a list: every mixture appends, per token, the gap between the logits of its last chosen and first unchosen expert


def mixture(h, mlp, w, p):
    r = mlp["router"]
    z = lin(w[p + "router"], h)
    scores = torch.softmax(z, dim=-1)
    if ROUTER_GAPS is not None and r["top"] < r["experts"]:
        ranked = z.sort(dim=-1, descending=True).values
        ROUTER_GAPS.append((ranked[:, r["top"] - 1] - ranked[:, r["top"]]).detach())
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = torch.topk(scores[t], r["top"]).indices.tolist()
        for e in chosen:
            out[t] += scores[t, e] * r["scale"] * expert(h[t], w, f"{p}e{e}.")
    if mlp.get("shared") is not None:
        out = out + expert(h, w, p + "shared.")
    return out


def feed_forward(h, mlp, w, p):
    if mlp["kind"] == "moe":
        return mixture(h, mlp, w, p)
    return expert(h, w, p)


# ------------------------------------------------------------------ the model

def layer_streams(tokens, cfg, w):
    """The residual stream after every layer, [layers, n, width]."""
    eps = cfg["norm"]["eps"]
    x = embed(tokens, w, (cfg.get("embedding") or {}).get("bigram"))
    kept = {}
    out = []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "attention":
            if m.get("kv_from") is None:
                kept[i] = attention_keys_values(x, m, w, p + "mix.", eps)
            y = attention_mixer(x, m, w, p + "mix.", eps, kept[m["kv_from"] if m.get("kv_from") is not None else i])
        elif layer["type"] == "latent_attention":
            y = latent_attention_mixer(x, m, w, p + "mix.", eps)
        elif layer["type"] == "mamba2":
            y = mamba2_mixer(x, m, w, p + "mix.", eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_unit(y, eps) * w[p + "norm1"] * w[p + "ls1"]
        if layer.get("mlp") is not None:
            x = x + rms_unit(feed_forward(x, layer["mlp"], w, p + "mlp."), eps) * w[p + "norm2"] * w[p + "ls2"]
        out.append(x)
    return torch.stack(out)


def logits(tokens, cfg, w):
    """[n, vocab]: the logits at every position of one sequence."""
    x = layer_streams(tokens, cfg, w)[-1]
    z = lin(w["head"], rms_unit(x, cfg["norm"]["eps"]) * w["final.norm"])
    cap = cfg.get("logit_softcap")
    return z if not cap else cap * torch.tanh(z / cap)


def greedy(tokens, cfg, w, n_new):
    tokens = list(tokens)
    out = []
    for _ in range(n_new):
        t = int(torch.argmax(logits(tokens, cfg, w)[-1]))
        out.append(t)
        tokens.append(t)
    return out
