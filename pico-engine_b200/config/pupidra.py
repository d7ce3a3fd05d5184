"""Typed configuration of the Pupidra decoder, read from its own config.json keys.

The design: the embedded token plus a row of a bigram table chosen by (previous token, token); layers whose sublayers
read the residual stream as it is and whose outputs are RMS-normed and multiplied by a learned vector before they are
added: ``x += ls1 * norm1(mixer(x)); x += ls2 * norm2(ff(x))``.  Each layer names its mixer: ``"attention"`` (grouped
softmax attention with biases, unit-normed queries and keys, a distance bias slope_h (i - j) with slope_h = 2^(-8 (h+1) / H),
a sliding window that keeps a sequence's first keys visible; with ``kv_from`` the layer has no key and value projections
and reads those of an earlier layer), ``"latent_attention"`` (keys and values from one low-rank row per position, one shared
rotated key part, pair rotation, a sigmoid gate a head) or ``"mamba2"`` (a selective state-space mixer).  The feed-forward
is a mixture of experts ``down(relu(up h)^2)`` weighted by their softmax scores over all experts times a factor, plus a
shared expert; or one such expert alone (``"dense"``); or absent.  A final RMS norm, the head, and a soft cap on the logits.
Every size and every constant that may differ between models comes from config.json:

    {"architecture": "Pupidra", "vocab": V, "width": W, "norm": {"eps": e}, "logit_softcap": c,
     "embedding": {"bigram": {"buckets", "mul_prev", "mul_cur"}},
     "layers": [{"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size", "keep_first"},
                 "kv_from": j}, "mlp": ...},
                {"type": "latent_attention", "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale",
                 "rot": {"base", "dims"}}, "mlp": ...},
                {"type": "mamba2", "mixer": {"heads", "vdim", "state", "groups", "conv", "norm_groups"}, "mlp": ...}]}
    mlp: null | {"kind": "dense", "ff": F} | {"kind": "moe", "router": {"experts", "top", "scale"}, "expert": {"ff"}, "shared": {"ff"}}
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

from .registry import register_architecture
from .specs import (BigramTableSpec, ConfigError, DenseMLPSpec, GatedAttentionSpec, LatentAttentionSpec, LayerSpec, MixtureSpec,
                    ModelPlan, NoPositionSpec, RMSNormSpec, RotaryPairsSpec, ScheduleEntry, StateSpaceSpec)

# Positions enter float32 angles and distances: every integer below 2^24 is exact there.
MAX_POSITIONS = 1 << 24


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


def distance_slopes(heads: int) -> Tuple[float, ...]:
    """The design's slope of head h of H: 2^(-8 (h + 1) / H)."""
    return tuple(2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads))


def _attention(m: dict, where: str, i: int) -> dict:
    out = {"heads": _int(m, "heads", where), "kv_heads": _int(m, "kv_heads", where), "dim": _int(m, "dim", where),
           "vdim": _int(m, "vdim", where), "scale": _number(m, "scale", where)}
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"{where}: {out['heads']} heads cannot share {out['kv_heads']} key/value heads evenly")
    if m.get("mask") is not None:
        mask = {"size": _int(m["mask"], "size", where + "mask.")}
        if m["mask"].get("keep_first") is not None:
            mask["keep_first"] = _int(m["mask"], "keep_first", where + "mask.", least=0)
        out["mask"] = mask
    if m.get("kv_from") is not None:
        out["kv_from"] = _int(m, "kv_from", where, least=0)
        if out["kv_from"] >= i:
            raise ConfigError(f"{where}kv_from = {out['kv_from']} must name an earlier layer than {i}")
    return out


def _latent(m: dict, where: str) -> dict:
    out = {k: _int(m, k, where) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank")}
    out["scale"] = _number(m, "scale", where)
    rot = m.get("rot")
    if not isinstance(rot, dict):
        raise ConfigError(f"{where}rot must be an object with base and dims")
    out["rot"] = {"base": _number(rot, "base", where + "rot."), "dims": _int(rot, "dims", where + "rot.")}
    if out["rot"]["dims"] % 2 or out["rot"]["dims"] > out["rot_dim"]:
        raise ConfigError(f"{where}rot.dims must be even and at most rot_dim = {out['rot_dim']}, found {out['rot']['dims']}")
    return out


def _mamba2(m: dict, where: str) -> dict:
    out = {k: _int(m, k, where) for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups")}
    if out["heads"] % out["groups"]:
        raise ConfigError(f"{where}: {out['heads']} heads cannot share {out['groups']} groups evenly")
    if (out["heads"] * out["vdim"]) % out["norm_groups"]:
        raise ConfigError(f"{where}norm_groups = {out['norm_groups']} does not divide heads * vdim = {out['heads'] * out['vdim']}")
    return out


def _mlp(mlp, where: str) -> Optional[dict]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"{where}kind must be \"dense\" or \"moe\" (or mlp null), found {mlp!r}")
    if mlp["kind"] == "dense":
        return {"ff": _int(mlp, "ff", where), "kind": "dense"}
    router = mlp.get("router")
    out = {"expert": {"ff": _int(mlp.get("expert"), "ff", where + "expert.")}, "kind": "moe",
           "router": {"experts": _int(router, "experts", where + "router."), "top": _int(router, "top", where + "router."),
                      "scale": _number(router, "scale", where + "router.") if isinstance(router, dict) and router.get("scale") is not None else 1.0}}
    if out["router"]["top"] > out["router"]["experts"]:
        raise ConfigError(f"{where}router.top = {out['router']['top']} exceeds router.experts = {out['router']['experts']}")
    if mlp.get("shared") is not None:
        out["shared"] = {"ff": _int(mlp["shared"], "ff", where + "shared.")}
    return out


@dataclass(frozen=True)
class PupidraLayer:
    """One entry of ``layers``: ``kind`` and the checked ``mixer`` and ``mlp`` objects as config.json spells them."""
    kind: str
    mixer: dict = field(hash=False)
    mlp: Optional[dict] = field(default=None, hash=False)

    @classmethod
    def from_dict(cls, d: dict, i: int) -> "PupidraLayer":
        where = f"layers[{i}]."
        if not isinstance(d, dict) or "type" not in d:
            raise ConfigError(f"layers[{i}] needs a type")
        kind, m = d["type"], d.get("mixer")
        if not isinstance(m, dict):
            raise ConfigError(f"{where}mixer must be an object with the mixer's sizes")
        mlp = _mlp(d.get("mlp"), where + "mlp.")
        if kind == "attention":
            return cls(kind, _attention(m, where + "mixer.", i), mlp)
        if kind == "latent_attention":
            return cls(kind, _latent(m, where + "mixer."), mlp)
        if kind == "mamba2":
            return cls(kind, _mamba2(m, where + "mixer."), mlp)
        raise ConfigError(f"{where}type must be \"attention\", \"latent_attention\" or \"mamba2\", found {kind!r}")

    def to_dict(self) -> dict:
        return {"mixer": dict(self.mixer), "mlp": self.mlp, "type": self.kind}


@dataclass(frozen=True)
class PupidraConfig:
    ARCHITECTURE = "Pupidra"

    vocab: int
    width: int
    layers: Tuple[PupidraLayer, ...]
    norm_eps: float
    bigram: Optional[Tuple[int, int, int]] = None      # (buckets, mul_prev, mul_cur)
    logit_softcap: Optional[float] = None

    @classmethod
    def from_dict(cls, d: dict) -> "PupidraConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm") if d.get(k) is None]
        if missing:
            raise ConfigError("config.json lacks " + ", ".join(missing))
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("layers must be a non-empty list")
        if not isinstance(d["norm"], dict):
            raise ConfigError("norm must be an object ({\"eps\": ...})")
        layers = tuple(PupidraLayer.from_dict(x, i) for i, x in enumerate(d["layers"]))
        for i, x in enumerate(layers):
            j = x.mixer.get("kv_from") if x.kind == "attention" else None
            if j is not None:
                src = layers[j]
                if src.kind != "attention" or src.mixer.get("kv_from") is not None:
                    raise ConfigError(f"layers[{i}].mixer.kv_from = {j} must name an attention layer with keys and values of its own")
                if any(src.mixer[k] != x.mixer[k] for k in ("kv_heads", "dim", "vdim")):
                    raise ConfigError(f"layers[{i}].mixer reads the keys and values of layer {j}: kv_heads, dim and vdim must be equal")
        big = (d.get("embedding") or {}).get("bigram")
        if big is not None:
            big = (_int(big, "buckets", "embedding.bigram."), _int(big, "mul_prev", "embedding.bigram.", least=0),
                   _int(big, "mul_cur", "embedding.bigram.", least=0))
        cap = d.get("logit_softcap")
        if cap is not None and (isinstance(cap, bool) or not isinstance(cap, (int, float)) or cap < 0):
            raise ConfigError(f"logit_softcap must be a positive number or absent, found {cap!r}")
        return cls(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""), layers=layers,
                   norm_eps=_number(d["norm"], "eps", "norm."), bigram=big, logit_softcap=float(cap) if cap else None)

    def to_dict(self) -> dict:
        d = {"architecture": self.ARCHITECTURE, "layers": [x.to_dict() for x in self.layers], "norm": {"eps": self.norm_eps},
             "vocab": self.vocab, "width": self.width}
        if self.bigram is not None:
            d["embedding"] = {"bigram": {"buckets": self.bigram[0], "mul_cur": self.bigram[2], "mul_prev": self.bigram[1]}}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        return d

    # ---------------------------------------------------------------- the plan

    @staticmethod
    def _mask(m: dict):
        mask = m.get("mask")
        return (None, 0) if mask is None else (mask["size"], mask.get("keep_first", 0))

    def _cache_span(self, i: int):
        """(window, keep_first) that layer i's cache must keep: what it and every layer that reads its keys and values can see."""
        spans = [self._mask(x.mixer) for j, x in enumerate(self.layers)
                 if x.kind == "attention" and (j == i or x.mixer.get("kv_from") == i)]
        window = None if any(w is None for w, _ in spans) else max(w for w, _ in spans)
        return window, (0 if window is None else max(f for _, f in spans))

    def _mixer_spec(self, i: int, x: PupidraLayer, p: str):
        W, eps, m = self.width, self.norm_eps, x.mixer
        if x.kind == "attention":
            window, keep = self._mask(m)
            own = m.get("kv_from") is None
            return GatedAttentionSpec(hidden=W, n_heads=m["heads"], n_kv_heads=m["kv_heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
                                      window=window, scale=m["scale"], position=NoPositionSpec(), prefix=p, qk_unit_norm=True,
                                      norm_eps=eps, gate=None, keep_first=keep if window is not None else 0,
                                      distance_slopes=distance_slopes(m["heads"]), bias=True, own_kv=own,
                                      cache_span=self._cache_span(i) if own else None)
        if x.kind == "latent_attention":
            return LatentAttentionSpec(hidden=W, n_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"], v_head_dim=m["vdim"],
                                       kv_rank=m["kv_rank"], scale=m["scale"],
                                       position=RotaryPairsSpec(head_dim=m["rot_dim"], dims=m["rot"]["dims"], base=m["rot"]["base"]),
                                       prefix=p, norm_eps=eps)
        return StateSpaceSpec(hidden=W, n_heads=m["heads"], head_dim=m["vdim"], state=m["state"], n_groups=m["groups"],
                              taps=m["conv"], norm_groups=m["norm_groups"], prefix=p, norm_eps=eps)

    def _ff_spec(self, mlp: Optional[dict], p: str):
        if mlp is None:
            return None
        if mlp["kind"] == "dense":
            return DenseMLPSpec(self.width, mlp["ff"], p, activation="relu2")
        shared = mlp.get("shared")
        return MixtureSpec(hidden=self.width, n_experts=mlp["router"]["experts"], top_k=mlp["router"]["top"],
                           intermediate=mlp["expert"]["ff"], prefix=p, activation="relu2",
                           shared_intermediate=None if shared is None else shared["ff"], shared_gate_name=None, gated=False,
                           scores="softmax_all", route_scale=mlp["router"]["scale"])

    def plan(self) -> ModelPlan:
        W, eps = self.width, self.norm_eps
        layers, schedule = [], []
        for i, x in enumerate(self.layers):
            p = f"l{i}."
            ff = self._ff_spec(x.mlp, p + "mlp.")
            layers.append(LayerSpec(mixer=self._mixer_spec(i, x, p + "mix."), mixer_norm=RMSNormSpec(W, eps, p + "norm1"),
                                    feed_forward=ff, feed_forward_norm=None if ff is None else RMSNormSpec(W, eps, p + "norm2"),
                                    arrangement="post_norm", mixer_scale=p + "ls1", feed_forward_scale=None if ff is None else p + "ls2"))
            schedule.append(ScheduleEntry(i, cache_of=x.mixer.get("kv_from") if x.kind == "attention" else None))
        # A layer without a feed-forward may still store its second norm and scale.
        unused = tuple(f"l{i}.{n}" for i, x in enumerate(self.layers) if x.mlp is None for n in ("norm2", "ls2"))
        plan = ModelPlan(architecture=self.ARCHITECTURE, vocab_size=self.vocab, hidden_size=W, embedding="embed",
                         layers=tuple(layers), schedule=tuple(schedule), final_norm=RMSNormSpec(W, eps, "final.norm"), head="head",
                         max_positions=MAX_POSITIONS, ignorable_tensors=unused, logit_softcap=self.logit_softcap,
                         embedding_pairs=None if self.bigram is None else BigramTableSpec(W, *self.bigram))
        plan.validate()
        return plan


register_architecture(PupidraConfig.ARCHITECTURE, PupidraConfig)
