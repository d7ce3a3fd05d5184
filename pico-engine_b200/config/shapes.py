"""config.json contents of the shapes the benchmarks and tests name: the two tiny test
configurations, the Qwen2.5 sizes and Mebalorn, Kevelorn, Pupidra and Tenusun models at the same widths (weights for them are drawn at random)."""
from __future__ import annotations

_QWEN2 = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_act": "silu", "torch_dtype": "bfloat16"}

SHAPES = {
    "tiny-a": {**_QWEN2, "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
               "head_dim": 16, "intermediate_size": 160, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
               "max_position_embeddings": 128, "tie_word_embeddings": True, "use_sliding_window": False},
    "tiny-b": {**_QWEN2, "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
               "head_dim": 32, "intermediate_size": 352, "vocab_size": 512, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
               "max_position_embeddings": 256, "tie_word_embeddings": False, "use_sliding_window": True,
               "sliding_window": 32, "max_window_layers": 1},
    "qwen2.5-0.5b": {**_QWEN2, "num_hidden_layers": 24, "hidden_size": 896, "num_attention_heads": 14,
                     "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 4864, "vocab_size": 151936,
                     "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 32768,
                     "tie_word_embeddings": True, "use_sliding_window": False},
    "qwen2.5-7b": {**_QWEN2, "num_hidden_layers": 28, "hidden_size": 3584, "num_attention_heads": 28,
                   "num_key_value_heads": 4, "head_dim": 128, "intermediate_size": 18944, "vocab_size": 152064,
                   "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 32768,
                   "tie_word_embeddings": False, "use_sliding_window": False},
    "qwen2.5-14b": {**_QWEN2, "num_hidden_layers": 48, "hidden_size": 5120, "num_attention_heads": 40,
                    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 13824, "vocab_size": 152064,
                    "rope_theta": 1000000.0, "rms_norm_eps": 1e-5, "max_position_embeddings": 32768,
                    "tie_word_embeddings": False, "use_sliding_window": False},
}


def mebalorn_shape(width: int, heads: int, kv_heads: int, dim: int, ff: int, layers: int, vocab: int, taps: int = 4,
                   vdim: int | None = None, softcap: float | None = 30.0) -> dict:
    """A Mebalorn config.json: recurrent and attention layers in turn (the first is recurrent), every layer with a
    feed-forward, the recurrent state as wide as the model."""
    att = {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim or dim, "scale": dim ** -0.5},
           "mlp": {"kind": "dense", "ff": ff}}
    rec = {"type": "mingru", "mixer": {"width": width}, "mlp": {"kind": "dense", "ff": ff}}
    d = {"architecture": "Mebalorn", "vocab": vocab, "width": width, "canon": {"taps": taps}, "norm": {"eps": 1e-6},
         "layers": [dict(rec if i % 2 == 0 else att) for i in range(layers)]}
    if softcap:
        d["logit_softcap"] = softcap
    return d


SHAPES.update({
    "mebalorn-tiny": mebalorn_shape(64, 4, 2, 16, 160, 4, 256, taps=3, vdim=32),
    "mebalorn-0.5b": mebalorn_shape(896, 14, 2, 64, 4864, 24, 151936),          # the widths of qwen2.5-0.5b
    "mebalorn-7b": mebalorn_shape(3584, 28, 4, 128, 18944, 28, 152064),         # the widths of qwen2.5-7b
})


def kevelorn_shape(width: int, heads: int, kv_heads: int, dim: int, ff: int, layers: int, vocab: int, window: int = 1024,
                   experts: int = 8, top: int = 2) -> dict:
    """A Kevelorn config.json whose layers take these four forms in turn: fixed-decay linear attention + dense feed-forward,
    learned-decay linear attention + mixture, windowed softmax attention beside linear attention + dense, fixed-decay linear
    attention + mixture.  Experts and the shared expert are a quarter as wide as the dense feed-forward."""
    decay = lambda n: [1.0 - 2.0 ** -(3 + h % 6) for h in range(n)]
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff // 4}, "shared": {"ff": ff // 4}}
    lightning = {"heads": heads, "dim": dim, "vdim": dim, "decay": decay(heads)}
    half = {"heads": max(heads // 2, 1), "dim": dim, "vdim": dim, "decay": decay(max(heads // 2, 1))}
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "mask": {"size": window},
            "rot": {"base": 10000.0, "dims": dim, "scaling": {"factor": 4.0}}}
    forms = [{"type": "lightning", "mixer": lightning, "mlp": dense},
             {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": dim, "tau": 16.0}, "mlp": moe},
             {"type": "parallel", "mixer": {"left": left, "right": half}, "mlp": dense},
             {"type": "lightning", "mixer": lightning, "mlp": moe}]
    return {"architecture": "Kevelorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "layers": [dict(forms[i % 4]) for i in range(layers)]}


SHAPES.update({
    "kevelorn-tiny": kevelorn_shape(64, 4, 2, 16, 160, 4, 256, window=40, experts=4),
    "kevelorn-0.5b": kevelorn_shape(896, 14, 2, 64, 4864, 24, 151936),          # the widths of qwen2.5-0.5b
    "kevelorn-7b": kevelorn_shape(3584, 28, 4, 128, 18944, 28, 152064),         # the widths of qwen2.5-7b
})


def pupidra_shape(width: int, heads: int, kv_heads: int, dim: int, ff: int, layers: int, vocab: int, window: int = 1024,
                  keep_first: int = 64, experts: int = 8, top: int = 2, state: int = 128, buckets: int = 16381) -> dict:
    """A Pupidra config.json whose layers take these four forms in turn: windowed attention with kept first keys and keys and
    values of its own, the state-space mixer (twice the width inside, heads of 64, two groups), latent attention (a cached row
    of at most 256 entries: rank 2 dim or 256 - dim / 2, rotated part dim / 2), and an attention that reads the first form's
    keys and values.  Every layer has a mixture whose experts and shared expert are a quarter as wide as a dense feed-forward."""
    moe = {"kind": "moe", "router": {"experts": experts, "top": top, "scale": 2.0}, "expert": {"ff": ff // 4}, "shared": {"ff": ff // 4}}
    att = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
           "mask": {"size": window, "keep_first": keep_first}}
    rot = max(2, dim // 2)
    rank = min(2 * dim, 256 - rot)
    lat = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": dim, "kv_rank": rank, "scale": (dim + rot) ** -0.5,
           "rot": {"base": 100000.0, "dims": rot}}
    p = min(64, 2 * width)
    ssm = {"heads": 2 * width // p, "vdim": p, "state": state, "groups": 2 if (2 * width // p) % 2 == 0 else 1, "conv": 4,
           "norm_groups": 2 if (2 * width // p) % 2 == 0 else 1}
    out = []
    for i in range(layers):
        form = i % 4
        mixer = (att, ssm, lat, {**att, "kv_from": i - 3})[form]
        out.append({"type": ("attention", "mamba2", "latent_attention", "attention")[form], "mixer": dict(mixer), "mlp": moe})
    return {"architecture": "Pupidra", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "logit_softcap": 30.0,
            "embedding": {"bigram": {"buckets": buckets, "mul_prev": 37, "mul_cur": 11}}, "layers": out}


SHAPES.update({
    "pupidra-tiny": pupidra_shape(64, 4, 2, 16, 160, 4, 256, window=40, keep_first=3, experts=4, state=24, buckets=97),
    "pupidra-0.5b": pupidra_shape(896, 14, 2, 64, 4864, 24, 151936),            # the widths of qwen2.5-0.5b
    "pupidra-7b": pupidra_shape(3584, 28, 4, 128, 18944, 28, 152064),           # the widths of qwen2.5-7b
})


def tenusun_shape(width: int, heads: int, kv_heads: int, dim: int, ff: int, layers: int, vocab: int, window: int = 1024,
                  experts: int = 8, top: int = 2, groups=(4, 2), vdim: int | None = None) -> dict:
    """A Tenusun config.json whose layers take these two forms in turn: latent attention behind a sliding window (a cached row of at
    most 256 entries: rank 2 dim or 256 - dim / 2, rotated part dim / 2, a query row a quarter of the width) with the dense clamped
    feed-forward, and grouped attention (half of a head rotated, stretched fourfold; values blended from the second such layer on)
    with a mixture whose experts are a quarter as wide as the dense feed-forward."""
    rot = max(2, dim // 2)
    rank = min(2 * dim, 256 - rot)
    lat = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": dim, "kv_rank": rank, "q_rank": max(64, width // 4 // 64 * 64),
           "scale": (dim + rot) ** -0.5, "rot": {"base": 500000.0, "dims": rot}, "mask": {"size": window}}
    att = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim or dim, "scale": dim ** -0.5, "v_mix": True,
           "rot": {"base": 500000.0, "dims": rot, "scaling": {"factor": 4.0, "original": 8192, "fast": 16.0, "slow": 2.0}}}
    dense = {"kind": "dense", "ff": ff, "limit": 7.0}
    moe = {"kind": "moe", "router": {"experts": experts, "top": top, "groups": {"count": groups[0], "keep": groups[1]}}, "expert": {"ff": ff // 4}}
    out = [{"type": "latent_attention", "mixer": dict(lat), "mlp": dict(dense)} if i % 2 == 0 else
           {"type": "attention", "mixer": dict(att), "mlp": dict(moe)} for i in range(layers)]
    return {"architecture": "Tenusun", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": float(width) ** 0.5},
            "layers": out}


SHAPES.update({
    "tenusun-tiny": tenusun_shape(64, 4, 2, 16, 160, 4, 256, window=40, experts=4, groups=(2, 1), vdim=8),
    "tenusun-0.5b": tenusun_shape(896, 14, 2, 64, 4864, 24, 151936),            # the widths of qwen2.5-0.5b
    "tenusun-7b": tenusun_shape(3584, 28, 4, 128, 18944, 28, 152064),           # the widths of qwen2.5-7b
})


def with_layers(d: dict, n: int) -> dict:
    """The shape with only its first ``n`` layers."""
    d = dict(d)
    if isinstance(d.get("layers"), list):
        d["layers"] = d["layers"][:n]
    else:
        d["num_hidden_layers"] = n
        d["max_window_layers"] = min(d.get("max_window_layers", n), n)
    return d


def shape(name: str) -> dict:
    try:
        return dict(SHAPES[name.lower()])
    except KeyError:
        raise KeyError(f"unknown shape {name!r}; known: {', '.join(sorted(SHAPES))}") from None
