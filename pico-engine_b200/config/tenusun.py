"""Typed configuration of the Tenusun decoder, read from its own config.json keys.

The design: the embedded token times ``embedding.scale``; layers with a layer norm (weight and bias) before and after each
sublayer, ``x += norm1b(mixer(norm1(x))); x += norm2b(ff(norm2(x)))``.  Each layer names its mixer: ``"latent_attention"``
(queries through a normed low-rank row, keys and values from another one, one rotated key part that all heads share, rotation
in the layout of halves, a sliding window, plain softmax) or ``"attention"`` (grouped attention whose keys and values may
differ in size, rotation of the first ``rot.dims`` entries in the layout of halves with frequencies stretched by ``rot.scaling``,
every earlier key visible, a softmax whose denominator has one added, values blended with those of the first ``v_mix`` layer,
a sigmoid gate on the concatenated heads).  The feed-forward is dense, ``down(g sigmoid(1.702 g) (u + 1))`` with
g = min(gate h, limit) and u = clamp(up h, -limit, limit); or a mixture of gated silu experts chosen by sigmoid scores plus a
stored correction among the best groups of experts, weighted by their plain scores; or absent.  A final layer norm, and the
embedding table as it is stored as the head.  Every size and every constant that may differ between models comes from config.json:

    {"architecture": "Tenusun", "vocab": V, "width": W, "norm": {"eps": e}, "embedding": {"scale": s},
     "layers": [{"type": "latent_attention", "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale",
                 "rot": {"base", "dims"}, "mask": {"size"}}, "mlp": ...},
                {"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "v_mix",
                 "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}}}, "mlp": ...}]}
    mlp: null | {"kind": "dense", "ff": F, "limit": l}
       | {"kind": "moe", "router": {"experts", "top", "groups": {"count", "keep"}}, "expert": {"ff"}}
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

from .registry import register_architecture
from .specs import (ConfigError, GatedAttentionSpec, GatedMLPSpec, LatentAttentionSpec, LayerNormSpec, LayerSpec, MixtureSpec,
                    ModelPlan, RotaryHalvesSpec, ScheduleEntry)

# Positions enter float32 angles: every integer below 2^24 is exact there.
MAX_POSITIONS = 1 << 24

# What the design fixes: the slope of the sigmoid in the dense feed-forward's activation, how many of a group's largest
# choice scores make the group's count, the score of the softmax's extra place, the factor's share in the size of cos and sin.
DENSE_ALPHA = 1.702
GROUP_BEST = 2
SINK_SCORE = 0.0
MAGNITUDE_SLOPE = 0.1


def _int(d, key: str, where: str, least: int = 1) -> int:
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, int) or v < least:
        raise ConfigError(f"{where}{key} must be an integer of at least {least}, found {v!r}")
    return v


def _number(d, key: str, where: str) -> float:
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not v > 0:
        raise ConfigError(f"{where}{key} must be a positive number, found {v!r}")
    return float(v)


def _rot(m: dict, where: str, most: int, stretch: bool) -> dict:
    rot = m.get("rot")
    if not isinstance(rot, dict):
        raise ConfigError(f"{where}rot must be an object with base and dims")
    out = {"base": _number(rot, "base", where + "rot."), "dims": _int(rot, "dims", where + "rot.", least=0)}
    if out["dims"] % 2 or out["dims"] > most:
        raise ConfigError(f"{where}rot.dims must be even and at most {most}, found {out['dims']}")
    sc = rot.get("scaling")
    if sc is not None:
        if not stretch:
            raise ConfigError(f"{where}rot.scaling: this mixer's rotation is not stretched")
        out["scaling"] = {k: _number(sc, k, where + "rot.scaling.") for k in ("factor", "original", "fast", "slow")}
        if out["base"] == 1.0:
            raise ConfigError(f"{where}rot.base = 1 leaves nothing to stretch")
    return out


def _latent(m: dict, where: str) -> dict:
    out = {k: _int(m, k, where) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank")}
    out["scale"] = _number(m, "scale", where)
    out["rot"] = _rot(m, where, out["rot_dim"], stretch=False)
    if m.get("mask") is not None:
        out["mask"] = {"size": _int(m["mask"], "size", where + "mask.")}
    return out


def _attention(m: dict, where: str) -> dict:
    out = {k: _int(m, k, where) for k in ("heads", "kv_heads", "dim", "vdim")}
    out["scale"] = _number(m, "scale", where)
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"{where}: {out['heads']} heads cannot share {out['kv_heads']} key/value heads evenly")
    out["rot"] = _rot(m, where, out["dim"], stretch=True)
    if m.get("v_mix") is not None:
        if not isinstance(m["v_mix"], bool):
            raise ConfigError(f"{where}v_mix must be true or false, found {m['v_mix']!r}")
        out["v_mix"] = m["v_mix"]
    return out


def _mlp(mlp, where: str) -> Optional[dict]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"{where}kind must be \"dense\" or \"moe\" (or mlp null), found {mlp!r}")
    if mlp["kind"] == "dense":
        return {"ff": _int(mlp, "ff", where), "kind": "dense", "limit": _number(mlp, "limit", where)}
    router = mlp.get("router")
    r = {"experts": _int(router, "experts", where + "router."), "top": _int(router, "top", where + "router.")}
    if r["top"] > r["experts"]:
        raise ConfigError(f"{where}router.top = {r['top']} exceeds router.experts = {r['experts']}")
    groups = router.get("groups")
    if groups is not None:
        g = {"count": _int(groups, "count", where + "router.groups."), "keep": _int(groups, "keep", where + "router.groups.")}
        if r["experts"] % g["count"]:
            raise ConfigError(f"{where}router.groups.count = {g['count']} does not divide router.experts = {r['experts']}")
        if g["keep"] > g["count"]:
            raise ConfigError(f"{where}router.groups.keep = {g['keep']} exceeds router.groups.count = {g['count']}")
        if g["keep"] * (r["experts"] // g["count"]) < r["top"]:
            raise ConfigError(f"{where}router.top = {r['top']} experts do not fit {g['keep']} group(s) of {r['experts'] // g['count']}")
        r["groups"] = g
    return {"expert": {"ff": _int(mlp.get("expert"), "ff", where + "expert.")}, "kind": "moe", "router": r}


@dataclass(frozen=True)
class TenusunLayer:
    """One entry of ``layers``: ``kind`` and the checked ``mixer`` and ``mlp`` objects as config.json spells them."""
    kind: str
    mixer: dict = field(hash=False)
    mlp: Optional[dict] = field(default=None, hash=False)

    @classmethod
    def from_dict(cls, d: dict, i: int) -> "TenusunLayer":
        where = f"layers[{i}]."
        if not isinstance(d, dict) or "type" not in d:
            raise ConfigError(f"layers[{i}] needs a type")
        kind, m = d["type"], d.get("mixer")
        if not isinstance(m, dict):
            raise ConfigError(f"{where}mixer must be an object with the mixer's sizes")
        mlp = _mlp(d.get("mlp"), where + "mlp.")
        if kind == "latent_attention":
            return cls(kind, _latent(m, where + "mixer."), mlp)
        if kind == "attention":
            return cls(kind, _attention(m, where + "mixer."), mlp)
        raise ConfigError(f"{where}type must be \"latent_attention\" or \"attention\", found {kind!r}")

    def to_dict(self) -> dict:
        return {"mixer": dict(self.mixer), "mlp": self.mlp, "type": self.kind}


@dataclass(frozen=True)
class TenusunConfig:
    ARCHITECTURE = "Tenusun"

    vocab: int
    width: int
    layers: Tuple[TenusunLayer, ...]
    norm_eps: float
    embedding_scale: float = 1.0

    @classmethod
    def from_dict(cls, d: dict) -> "TenusunConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm") if d.get(k) is None]
        if missing:
            raise ConfigError("config.json lacks " + ", ".join(missing))
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("layers must be a non-empty list")
        if not isinstance(d["norm"], dict):
            raise ConfigError("norm must be an object ({\"eps\": ...})")
        emb = d.get("embedding")
        scale = 1.0 if not isinstance(emb, dict) or emb.get("scale") is None else _number(emb, "scale", "embedding.")
        layers = tuple(TenusunLayer.from_dict(x, i) for i, x in enumerate(d["layers"]))
        mixing = [x.mixer for x in layers if x.kind == "attention" and x.mixer.get("v_mix")]
        for m in mixing[1:]:
            if (m["kv_heads"], m["vdim"]) != (mixing[0]["kv_heads"], mixing[0]["vdim"]):
                raise ConfigError("layers that mix values must have the same kv_heads and vdim as the first of them")
        return cls(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""), layers=layers,
                   norm_eps=_number(d["norm"], "eps", "norm."), embedding_scale=scale)

    def to_dict(self) -> dict:
        return {"architecture": self.ARCHITECTURE, "embedding": {"scale": self.embedding_scale},
                "layers": [x.to_dict() for x in self.layers], "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}

    # ---------------------------------------------------------------- the plan

    def _first_mixing(self) -> Optional[int]:
        return next((i for i, x in enumerate(self.layers) if x.kind == "attention" and x.mixer.get("v_mix")), None)

    def _mixer_spec(self, i: int, x: TenusunLayer, p: str):
        W, eps, m = self.width, self.norm_eps, x.mixer
        rot = m["rot"]
        if x.kind == "latent_attention":
            return LatentAttentionSpec(hidden=W, n_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"], v_head_dim=m["vdim"],
                                       kv_rank=m["kv_rank"], scale=m["scale"],
                                       position=RotaryHalvesSpec(head_dim=m["rot_dim"], dims=rot["dims"], base=rot["base"]),
                                       prefix=p, norm_eps=eps, gate=None, window=(m.get("mask") or {}).get("size"), q_rank=m["q_rank"])
        sc = rot.get("scaling")
        position = RotaryHalvesSpec(head_dim=m["dim"], dims=rot["dims"], base=rot["base"],
                                    stretch=None if sc is None else (sc["factor"], sc["original"], sc["fast"], sc["slow"]),
                                    magnitude_slope=MAGNITUDE_SLOPE)
        role = None
        if m.get("v_mix"):
            role = "source" if i == self._first_mixing() else "reader"
        return GatedAttentionSpec(hidden=W, n_heads=m["heads"], n_kv_heads=m["kv_heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
                                  window=None, scale=m["scale"], position=position, prefix=p, norm_eps=eps, gate="g",
                                  fixed_sink=SINK_SCORE, value_blend="vmix" if role == "reader" else None, value_blend_role=role)

    def _ff_spec(self, mlp: Optional[dict], p: str):
        if mlp is None:
            return None
        if mlp["kind"] == "dense":
            return GatedMLPSpec(self.width, mlp["ff"], p, activation="clamped_sigmoid", limit=mlp["limit"], alpha=DENSE_ALPHA)
        r = mlp["router"]
        groups = r.get("groups") or {"count": 1, "keep": 1}
        return MixtureSpec(hidden=self.width, n_experts=r["experts"], top_k=r["top"], intermediate=mlp["expert"]["ff"], prefix=p,
                           activation="silu", shared_intermediate=None, scores="sigmoid", correction_name="correction",
                           n_groups=groups["count"], keep_groups=groups["keep"], group_best=GROUP_BEST)

    def plan(self) -> ModelPlan:
        W, eps = self.width, self.norm_eps

        def norm(name: str) -> LayerNormSpec:
            return LayerNormSpec(W, eps, name, name + ".b")
        layers, schedule, unused = [], [], []
        for i, x in enumerate(self.layers):
            p = f"l{i}."
            ff = self._ff_spec(x.mlp, p + "mlp.")
            layers.append(LayerSpec(mixer=self._mixer_spec(i, x, p + "mix."), mixer_norm=norm(p + "norm1"), feed_forward=ff,
                                    feed_forward_norm=None if ff is None else norm(p + "norm2"), arrangement="sandwich",
                                    mixer_out_norm=norm(p + "norm1b"), feed_forward_out_norm=None if ff is None else norm(p + "norm2b")))
            schedule.append(ScheduleEntry(i))
            if x.kind == "attention" and (not x.mixer.get("v_mix") or i == self._first_mixing()):
                unused.append(p + "mix.vmix")            # stored beside a layer that blends nothing: left unread
            if ff is None:                               # a layer without a feed-forward may still store its norms
                unused.extend(p + n for n in ("norm2", "norm2.b", "norm2b", "norm2b.b"))
        plan = ModelPlan(architecture=self.ARCHITECTURE, vocab_size=self.vocab, hidden_size=W, embedding="embed",
                         layers=tuple(layers), schedule=tuple(schedule), final_norm=norm("final.norm"), head=None,
                         max_positions=MAX_POSITIONS, ignorable_tensors=tuple(unused), embedding_scale=self.embedding_scale)
        plan.validate()
        return plan


register_architecture(TenusunConfig.ARCHITECTURE, TenusunConfig)
