"""Small Tenusun configurations and random weights for the tests, written out independently of the library.

The configurations differ from one another in every size and option: which mixer comes first; query heads per key/value head
(1, 2, 3, 8); keys larger than, equal to and smaller than values; rotation of all, half, a fifth and none of a head's entries,
stretched or not, with ramps that lie inside the entries, that collapse to a step behind the first entry, and that reach beyond the last; one, two and three layers that blend values, the
first of them at the front or not, and layers beside them that blend nothing; latent rows of every parity with windows of 1
and 2 tokens, below a cache page, exactly a page, above two pages, and none; query rows narrower and wider than the key rows;
experts with top 1, top = experts and in between, in 1, 2, 4 groups and a group an expert, of which 1, 2 or all stay, or without
groups; layers without a feed-forward; embedding scales including 1.  Weights have the scale 1/sqrt(inputs) so that
activations keep their size and scores spread.
"""
from __future__ import annotations

import torch


def latent(heads, dim, rot_dim, vdim, rank, q_rank, scale, base, window=None, rot_dims=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "q_rank": q_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    if window is not None:
        m["mask"] = {"size": window}
    return "latent_attention", m


def attention(heads, kv_heads, dim, vdim, scale, rot_dims, base, scaling=None, v_mix=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"base": base, "dims": rot_dims}}
    if scaling is not None:
        m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if v_mix is not None:
        m["v_mix"] = v_mix
    return "attention", m


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, groups=None):
    r = {"experts": experts, "top": top}
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "router": r, "expert": {"ff": ff}}


def layer(mixer, mlp):
    return {"type": mixer[0], "mixer": mixer[1], "mlp": mlp}


def config(vocab, width, eps, scale, layers):
    return {"architecture": "Tenusun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale}, "layers": layers}


CONFIGS = {
    # attention first; 3 query heads a key/value head, values smaller than keys, half of a head rotated with a ramp inside the
    # entries; three blending layers; a window below a page; 4 groups of 2 of which 2 stay, top 3; a layer without feed-forward
    "T1": config(300, 80, 1e-5, 3.0, [
        layer(attention(6, 2, 32, 16, 0.3, 16, 1000.0, (4.0, 64, 8.0, 2.0), v_mix=True), moe(8, 3, 24, (4, 2))),
        layer(latent(3, 24, 16, 40, 48, 40, 0.2, 1000.0, window=33), dense(96, 2.0)),
        layer(attention(4, 2, 48, 16, 0.2, 48, 300.0, v_mix=True), dense(64, 0.7)),
        layer(attention(6, 2, 32, 16, 0.25, 16, 1000.0, (4.0, 64, 8.0, 2.0), v_mix=True), moe(8, 3, 24, (4, 2))),
        layer(latent(3, 24, 16, 40, 48, 40, 0.2, 1000.0, window=70), None)]),
    # no window at all; one query head a key/value head, values larger than keys, every entry rotated, a ramp that is a step behind
    # the first entry (every other frequency divided), and one that reaches beyond the last; a layer that blends nothing in front of the two that do; top = experts without
    # groups, and one group; an embedding scale of 1
    "T2": config(128, 48, 1e-3, 1.0, [
        layer(attention(4, 4, 16, 24, 0.5, 16, 50.0, (2.0, 16, 64.0, 32.0)), moe(2, 2, 16)),
        layer(latent(2, 8, 8, 16, 40, 12, 0.35, 50.0), moe(4, 3, 16, (1, 1))),
        layer(attention(2, 1, 16, 24, 0.4, 8, 50.0, v_mix=True), dense(40, 5.0)),
        layer(attention(2, 1, 16, 24, 0.4, 8, 50.0, (16.0, 16, 1.0, 0.01), v_mix=True), moe(2, 2, 16))]),
    # sizes that are multiples of nothing: head sizes 24 / 12, ten rotated entries (five pairs), a cached latent row of 26 entries,
    # a width that is no multiple of 4; windows of 2 tokens, of 1 token and of exactly a page; a group an expert of which 3 stay;
    # one blending layer alone (it blends nothing); no rotation at all in one layer
    "T3": config(90, 50, 2e-6, 0.5, [
        layer(latent(5, 12, 6, 10, 20, 14, 0.3, 100.0, window=2), moe(6, 2, 20, (6, 3))),
        layer(attention(3, 1, 24, 12, 0.35, 10, 100.0, (8.0, 32, 4.0, 0.5), v_mix=True), moe(6, 1, 20, (3, 1))),
        layer(latent(2, 10, 4, 6, 9, 30, 0.4, 20.0, window=64), dense(36, 1.0)),
        layer(latent(2, 10, 4, 6, 9, 30, 0.4, 20.0, window=1), None),
        layer(attention(2, 2, 16, 16, 0.5, 0, 100.0), dense(36, 1.0))]),
    # sizes of the tensor-core kernels: head size 64 with 8 query heads on one key/value head and equal values, a window above
    # two pages, latent rows of 64 + 32, query rows wider than key rows; a blending layer behind a latent one; 2 groups of 4, 1 stays
    "T4": config(200, 128, 1e-5, 8.0, [
        layer(latent(4, 32, 32, 32, 64, 96, 0.11, 40000.0, window=130), moe(8, 2, 32, (2, 1))),
        layer(attention(8, 1, 64, 64, 0.125, 32, 40000.0, (8.0, 128, 16.0, 1.0), v_mix=True), dense(160, 1.25)),
        layer(attention(8, 1, 64, 64, 0.125, 32, 40000.0, (8.0, 128, 16.0, 1.0), v_mix=True), moe(8, 2, 32, (2, 1))),
        layer(latent(4, 32, 32, 32, 64, 96, 0.11, 40000.0, window=45), dense(160, 1.25))]),
}


def tensor_shapes(cfg: dict) -> dict:
    W, V = cfg["width"], cfg["vocab"]
    shapes = {"embed": (V, W), "final.norm": (W,), "final.norm.b": (W,)}
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", l["mixer"]
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if l["mlp"] is not None else ()):
            shapes[f"l{i}.{n}"] = (W,)
            shapes[f"l{i}.{n}.b"] = (W,)
        if l["type"] == "attention":
            H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            shapes.update({p + "q": (H * D, W), p + "k": (G * D, W), p + "v": (G * Dv, W), p + "g": (H * Dv, W), p + "o": (W, H * Dv)})
            if m.get("v_mix"):
                shapes[p + "vmix"] = ()
        else:
            H, D, R, Dv, rank, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            shapes.update({p + "dq": (qr, W), p + "dq.norm": (qr,), p + "uq": (H * (D + R), qr), p + "dkv": (rank + R, W),
                           p + "dkv.norm": (rank,), p + "uk": (H * D, rank), p + "uv": (H * Dv, rank), p + "o": (W, H * Dv)})
        mlp = l["mlp"]
        if mlp is None:
            continue
        q = f"l{i}.mlp."
        if mlp["kind"] == "dense":
            shapes.update({q + "gate": (mlp["ff"], W), q + "up": (mlp["ff"], W), q + "down": (W, mlp["ff"])})
            continue
        E, F = mlp["router"]["experts"], mlp["expert"]["ff"]
        shapes[q + "router"] = (E, W)
        shapes[q + "correction"] = (E,)
        for e in range(E):
            shapes.update({f"{q}e{e}.gate": (F, W), f"{q}e{e}.up": (F, W), f"{q}e{e}.down": (W, F)})
    return shapes


def steady_correction(experts: int, groups, g) -> torch.Tensor:
    """Corrections half a unit apart in a random order, drawn again until the groups' counts (the sum of a group's two largest)
    lie at least 0.45 apart: with scores that stay near one half, no choice of a group or an expert is ever a close call."""
    while True:
        c = (torch.randperm(experts, generator=g).float() - experts / 3.0) * 0.5 + 0.04 * torch.rand(experts, generator=g)
        if groups is None or groups["count"] == 1:
            return c
        sums = sorted(float(torch.sort(part, descending=True).values[:2].sum()) for part in c.view(groups["count"], -1))
        if min(b - a for a, b in zip(sums, sums[1:])) >= 0.45:
            return c


def make_weights(cfg: dict, seed: int, steady_routing: bool = False) -> dict:
    """Random weights rounded to bfloat16 values (kept in float32 here).  ``steady_routing``: routers whose scores stay within a
    tenth of one half and corrections that decide every choice by a wide margin (for runs in bfloat16, where a choice that
    rounding can turn would change a token's feed-forward and, through the attention layers behind it, every later position);
    otherwise scores and corrections of comparable spread, so that the choice varies from token to token."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if steady_routing and last in ("router", "correction"):
            r = cfg["layers"][int(name.split(".")[0][1:])]["mlp"]["router"]
            t = torch.randn(shape, generator=g) * 0.2 * shape[1] ** -0.5 if last == "router" else steady_correction(r["experts"], r.get("groups"), g)
            out[name] = t.to(torch.bfloat16).to(torch.float32)
            continue
        if last in ("norm1", "norm2", "norm1b", "norm2b", "norm"):
            t = (0.5 if last.endswith("b") else 1.0) + 0.1 * torch.randn(shape, generator=g)
        elif last == "b":
            t = 0.2 * torch.randn(shape, generator=g)
        elif last == "router":
            t = torch.randn(shape, generator=g) * 1.5 * shape[1] ** -0.5      # logits about a unit apart: sigmoids that do not saturate
        elif last == "correction":
            t = torch.randn(shape, generator=g) - 0.3                          # choice scores of either sign, a few tenths apart
        elif last == "vmix":
            t = 0.25 + 0.5 * torch.rand(shape, generator=g)                    # a blend that shows
        elif name == "embed":
            t = torch.randn(shape, generator=g) * 0.7 / max(cfg["embedding"]["scale"], 1.0) ** 0.5
        else:
            t = torch.randn(shape, generator=g) * shape[1] ** -0.5
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out


def requests_for(cfg: dict, lengths, seed: int = 7) -> dict:
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}


_cache = {}
CLOSE_CALL = 0.03       # bfloat16 rounding of a router's input moves its scores (sigmoids: slope 1/4 at most) by a few thousandths


def plain_logits(cfg: dict, weights: dict, requests: dict, close_calls: set | None = None) -> dict:
    """{(request, position): logits row} of the plain implementation in float64 (kept: the tests ask for the same requests
    in several ways of cutting).  ``close_calls`` receives the (request, position) pairs at which some router of the plain run
    chose its last group or expert by less than CLOSE_CALL: there a run in bfloat16 may rightly choose another, and the
    comparison in bfloat16 leaves those places out (float32 runs are compared everywhere).  A choice made at a position also
    reaches later positions through the mixers, but only weakly; a close call is left out at its own position."""
    import plain_tenusun as plain
    out = {}
    w64 = None
    for rid, toks in requests.items():
        key = (id(weights), tuple(toks))
        if key not in _cache:
            if w64 is None:
                w64 = {n: t.double() for n, t in weights.items()}
            plain.ROUTER_GAPS = []
            with torch.no_grad():
                logits = plain.logits(cfg, w64, toks).float().numpy()
            gaps, plain.ROUTER_GAPS = plain.ROUTER_GAPS, None
            close = torch.stack(gaps).min(0).values < CLOSE_CALL if gaps else torch.zeros(len(toks), dtype=torch.bool)
            _cache[key] = (logits, close.tolist())
        logits, close = _cache[key]
        for p in range(len(toks)):
            out[(rid, p)] = logits[p]
            if close_calls is not None and close[p]:
                close_calls.add((rid, p))
    return out
