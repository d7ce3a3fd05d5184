"""Small Pupidra configurations and random weights for the tests, written out independently of the library.

The configurations differ from one another in every size and option: the order of the mixers; query heads per key/value
head (1, 2, 3, 8); key and value sizes (equal or not, multiples of 16 or of nothing); windows of 2 tokens, below a cache
page, exactly a page, above two pages, and none; kept first tokens 0, 1, a page, more than a page; layers that read
another layer's keys and values through another window; latent ranks and rotated parts of every parity, rotation of all or
of part of the rotated entries; state sizes from 7 to 128 with 1 to 4 groups, 1 to 4 taps, 1 to 4 norm groups; experts
with top 1, top = experts and in between, with and without a shared expert, router factors including 1; layers without a
feed-forward; a model without bigram rows or soft cap.  Weights have the scale 1/sqrt(inputs) so that activations keep
their size and scores spread.
"""
from __future__ import annotations

import torch


def attention(heads, kv_heads, dim, vdim, scale, mask=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if mask is not None:
        m["mask"] = {"size": mask[0], "keep_first": mask[1]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return "attention", m


def latent(heads, dim, rot_dim, vdim, rank, scale, rot_dims, base):
    return "latent_attention", {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
                                "rot": {"dims": rot_dims, "base": base}}


def mamba2(heads, vdim, state, groups, conv, norm_groups):
    return "mamba2", {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def moe(experts, top, scale, ff, shared=None):
    d = {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale}, "expert": {"ff": ff}}
    if shared is not None:
        d["shared"] = {"ff": shared}
    return d


def layer(mixer, mlp):
    return {"type": mixer[0], "mixer": mixer[1], "mlp": mlp}


def config(vocab, width, eps, layers, bigram=None, softcap=None):
    d = {"architecture": "Pupidra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if bigram is not None:
        d["embedding"] = {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}
    if softcap is not None:
        d["logit_softcap"] = softcap
    return d


CONFIGS = {
    # 3 query heads a key/value head, values smaller than keys, a window below a page with a few kept tokens; a reader of layer 0's
    # keys through a wider window without kept tokens; part of the rotated entries rotated; a layer without feed-forward
    "P1": config(300, 80, 1e-5, [
        layer(attention(6, 2, 32, 16, 0.3, mask=(40, 5)), moe(5, 2, 1.7, 24, 40)),
        layer(mamba2(4, 16, 24, 2, 3, 4), None),
        layer(latent(3, 24, 16, 40, 48, 0.2, 8, 1000.0), moe(3, 1, 1.0, 32)),
        layer(attention(6, 2, 32, 16, 0.25, mask=(70, 0), kv_from=0), moe(5, 2, 1.7, 24, 40))], bigram=(97, 13, 5), softcap=20.0),
    # no window at all; one query head a key/value head, values larger than keys; one group, one norm group, two taps;
    # top = experts; no bigram rows, no soft cap
    "P2": config(128, 48, 1e-3, [
        layer(mamba2(2, 8, 40, 1, 2, 1), moe(2, 2, 0.5, 16, 8)),
        layer(attention(4, 4, 16, 24, 0.5), moe(4, 3, 2.0, 16)),
        layer(latent(2, 8, 8, 16, 40, 0.35, 8, 50.0), None),
        layer(attention(4, 4, 16, 24, 0.4, kv_from=1), moe(2, 2, 0.5, 16, 8))]),
    # sizes that are multiples of nothing: head sizes 24 / 12, a cached latent row of 26 entries, a state of 7 rows, one tap,
    # groups = heads, a width that is no multiple of 4; windows of 2 tokens (1 kept) and of exactly a page (a page kept)
    "P3": config(90, 50, 2e-6, [
        layer(attention(3, 1, 24, 12, 0.35, mask=(2, 1)), moe(7, 3, 3.0, 20, 12)),
        layer(latent(5, 12, 6, 10, 20, 0.3, 6, 100.0), moe(7, 3, 3.0, 20, 12)),
        layer(mamba2(3, 5, 7, 3, 1, 3), moe(2, 1, 1.0, 36)),
        layer(attention(2, 2, 16, 16, 0.5, mask=(64, 64)), None)], bigram=(11, 3, 7), softcap=5.0),
    # sizes of the tensor-core kernels: head size 64 with 8 query heads on one key/value head, a window above two pages with more
    # than a page kept, two readers of one layer's keys; latent rows of 64 + 32; a state of 128 rows, four taps
    "P4": config(200, 128, 1e-5, [
        layer(mamba2(4, 32, 128, 4, 4, 2), moe(4, 2, 2.25, 32, 64)),
        layer(attention(8, 1, 64, 64, 0.125, mask=(130, 70)), moe(4, 2, 2.25, 32, 64)),
        layer(attention(8, 1, 64, 64, 0.125, mask=(130, 70), kv_from=1), None),
        layer(latent(4, 32, 32, 32, 64, 0.125, 32, 40000.0), moe(4, 2, 2.25, 32, 64)),
        layer(attention(8, 1, 64, 64, 0.2, mask=(33, 0), kv_from=1), moe(4, 2, 2.25, 32, 64))], bigram=(211, 29, 3), softcap=12.0),
}


def tensor_shapes(cfg: dict) -> dict:
    W, V = cfg["width"], cfg["vocab"]
    shapes = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    if cfg.get("embedding"):
        shapes["bigram"] = (cfg["embedding"]["bigram"]["buckets"] + 1, W)
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", l["mixer"]
        shapes[f"l{i}.norm1"] = (W,)
        shapes[f"l{i}.ls1"] = (W,)
        if l["type"] == "attention":
            H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            shapes.update({p + "q": (H * D, W), p + "q.b": (H * D,), p + "o": (W, H * Dv), p + "o.b": (W,)})
            if m.get("kv_from") is None:
                shapes.update({p + "k": (G * D, W), p + "k.b": (G * D,), p + "v": (G * Dv, W), p + "v.b": (G * Dv,)})
        elif l["type"] == "latent_attention":
            H, D, R, Dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            shapes.update({p + "q": (H * (D + R), W), p + "dkv": (rank + R, W), p + "dkv.norm": (rank,), p + "uk": (H * D, rank),
                           p + "uv": (H * Dv, rank), p + "g": (H, W), p + "o": (W, H * Dv)})
        else:
            H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            inner, conv = H * P, H * P + 2 * G * N
            shapes.update({p + "in": (2 * inner + 2 * G * N + H, W), p + "conv": (conv, m["conv"]), p + "conv.b": (conv,),
                           p + "dt_bias": (H,), p + "A_log": (H,), p + "D": (H,), p + "norm": (inner,), p + "o": (W, inner)})
        mlp = l["mlp"]
        if mlp is None:
            continue
        q = f"l{i}.mlp."
        shapes[f"l{i}.norm2"] = (W,)
        shapes[f"l{i}.ls2"] = (W,)
        experts = [(f"{q}e{e}.", mlp["expert"]["ff"]) for e in range(mlp["router"]["experts"])]
        if mlp.get("shared"):
            experts.append((q + "shared.", mlp["shared"]["ff"]))
        shapes[q + "router"] = (mlp["router"]["experts"], W)
        for e, F in experts:
            shapes.update({e + "up": (F, W), e + "down": (W, F)})
    return shapes


def make_weights(cfg: dict, seed: int) -> dict:
    """Random weights rounded to bfloat16 values (kept in float32 here)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm2", "norm") or name == "final.norm":
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif last in ("ls1", "ls2"):
            t = 0.5 + 0.2 * torch.rand(shape, generator=g)
        elif last == "router":
            t = torch.randn(shape, generator=g) * 4.0 * shape[1] ** -0.5      # logits several units apart: few close calls
        elif last == "b":
            t = 0.3 * torch.randn(shape, generator=g)
        elif last == "conv":
            t = torch.randn(shape, generator=g) * 0.6
        elif last == "dt_bias":
            t = torch.randn(shape, generator=g) - 1.0                          # step sizes from 0.05 to 1
        elif last == "A_log":
            t = torch.randn(shape, generator=g) * 0.7 - 0.5                    # decays a token from 0.3 to 0.98
        elif last == "D":
            t = 1.0 + 0.3 * torch.randn(shape, generator=g)
        elif name in ("embed", "bigram"):
            t = torch.randn(shape, generator=g) * 0.7
        else:
            t = torch.randn(shape, generator=g) * shape[1] ** -0.5
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out


def requests_for(cfg: dict, lengths, seed: int = 7) -> dict:
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}


_cache = {}
CLOSE_CALL = 0.1        # bfloat16 rounding of a router's input moves its logits by a few hundredths


def plain_logits(cfg: dict, weights: dict, requests: dict, close_calls: set | None = None) -> dict:
    """{(request, position): logits row} of the plain implementation in float64 (kept: the tests ask for the same requests
    in several ways of cutting).  ``close_calls`` receives the (request, position) pairs at which some router of the plain run
    chose its last expert by less than CLOSE_CALL: there a run in bfloat16 may rightly choose another expert, and the
    comparison in bfloat16 leaves those places out (float32 runs are compared everywhere).  A choice made at a position also
    reaches later positions through the mixers, but only weakly; a close call is left out at its own position."""
    import plain_pupidra as plain
    out = {}
    w64 = None
    for rid, toks in requests.items():
        key = (id(weights), tuple(toks))
        if key not in _cache:
            if w64 is None:
                w64 = {n: t.double() for n, t in weights.items()}
            plain.ROUTER_GAPS = []
            with torch.no_grad():
                logits = plain.logits(toks, cfg, w64).float().numpy()
            gaps, plain.ROUTER_GAPS = plain.ROUTER_GAPS, None
            close = torch.stack(gaps).min(0).values < CLOSE_CALL if gaps else torch.zeros(len(toks), dtype=torch.bool)
            _cache[key] = (logits, close.tolist())
        logits, close = _cache[key]
        for p in range(len(toks)):
            out[(rid, p)] = logits[p]
            if close_calls is not None and close[p]:
                close_calls.add((rid, p))
    return out
