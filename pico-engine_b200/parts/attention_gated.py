"""Grouped softmax attention with an output gate, optional unit norm of queries and keys, and its position encoding."""
from __future__ import annotations

import torch

from ..cache import CacheNeeds, KVNeed
import math

from ..config.specs import ConfigError, GatedAttentionSpec, NoPositionSpec, RotaryHalvesSpec, RotaryPairsSpec
from ..ops import kernels, linear
from ..weights.loader import ParamSpec
from .base import Mixer, first_product, last_product_into, normed_rows, register_mixer


def pair_frequencies(spec: RotaryPairsSpec, device) -> torch.Tensor:
    """base^(-2i/dims) / factor for i < dims / 2, worked out in float64 and rounded once to float32."""
    i = torch.arange(spec.dims // 2, dtype=torch.float64)
    return (spec.base ** (-2.0 * i / spec.dims) / spec.factor).to(torch.float32).to(device)


def halves_frequencies(spec: RotaryHalvesSpec, device):
    """(frequencies float32 [dims / 2], the factor on cos and sin) of a rotation in the layout of halves: base^(-2i/dims), each
    stretched by ``spec.stretch`` where that is given; worked out in float64 and rounded once to float32."""
    half = spec.dims // 2
    f = [spec.base ** (-2.0 * i / spec.dims) for i in range(half)]
    magnitude = 1.0
    if spec.stretch is not None and half:
        factor, original, fast, slow = spec.stretch

        def where(turns: float) -> float:
            return spec.dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(spec.base))
        lo = max(math.floor(where(fast)), 0)
        hi = min(math.ceil(where(slow)), spec.dims - 1)
        for i in range(half):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            f[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp)
        magnitude = spec.magnitude_slope * math.log(factor) + 1.0
    return torch.tensor(f, dtype=torch.float64).to(torch.float32).to(device), magnitude


@register_mixer(GatedAttentionSpec)
class GatedAttention(Mixer):
    """One product for q, k, v and the gate; rotation of neighbouring pairs of q and k, unit norm of every head and the
    cache write in one kernel (csrc/gated_ops.cu); attention over the cache (the kernels of grouped attention where keys
    and values have one size that they take, else the float32-score kernels that take any two sizes); the heads times
    sigmoid(gate); the output projection.  Angles, norms, scores, softmax and the gate are float32 in either dtype."""

    takes_out_dtype = True      # apply(..., out_dtype=) gives the product's float32 sums where the caller goes on in float32

    def __init__(self, spec: GatedAttentionSpec, dtype, device):
        super().__init__(spec, dtype, device)
        if spec.n_heads % spec.n_kv_heads:
            raise ConfigError(f"{spec.n_heads} query heads cannot share {spec.n_kv_heads} key/value heads evenly")
        if not isinstance(spec.position, (NoPositionSpec, RotaryPairsSpec, RotaryHalvesSpec)):
            raise ConfigError("gated attention takes rotation of pairs, of halves, or no position encoding")
        if isinstance(spec.position, RotaryHalvesSpec) and (spec.position.dims % 2 or spec.position.dims > spec.head_dim):
            raise ConfigError(f"{spec.position.dims} rotated entries do not fit a head of {spec.head_dim}")
        if spec.value_blend_role not in (None, "source", "reader") or (spec.value_blend_role == "reader") != (spec.value_blend is not None):
            raise ConfigError("value_blend_role is \"source\", \"reader\" (with the name of its number) or None")
        if spec.value_blend_role is not None and not (spec.own_kv and isinstance(spec.position, RotaryHalvesSpec)):
            raise ConfigError("values are blended in the kernel that rotates halves, for a mixer with keys and values of its own")
        if spec.head_dim > 256 or spec.v_head_dim > 256:
            raise ConfigError(f"head sizes {spec.head_dim}/{spec.v_head_dim} are not taken: up to 256 are")
        if spec.window is not None and spec.window <= 0:
            raise ConfigError(f"window {spec.window} must be positive")
        self.state_offset = 0
        if spec.distance_slopes is not None and len(spec.distance_slopes) != spec.n_heads:
            raise ConfigError(f"{len(spec.distance_slopes)} distance slopes for {spec.n_heads} heads")
        if spec.keep_first < 0 or (spec.keep_first and spec.window is None):
            raise ConfigError("keep_first belongs to a window and cannot be negative")
        self.w_in = self.w_o = self.freq = self.b_in = self.b_o = self.slopes = self.sink = self.blend_weight = None
        self.magnitude = 1.0
        # the kernels of grouped attention take equal key and value sizes: any up to 256 in float32, multiples of 16 in bfloat16;
        # a distance bias and kept first keys are known to the kernels that take two sizes
        self.plain_kernels = (spec.v_head_dim == spec.head_dim and (dtype == torch.float32 or spec.head_dim % 16 == 0)
                              and spec.distance_slopes is None and not spec.keep_first and spec.fixed_sink is None)

    def _widths(self):
        s = self.spec
        return s.n_heads * s.head_dim, s.n_kv_heads * s.head_dim, s.n_kv_heads * s.v_head_dim, s.n_heads * s.v_head_dim

    def _in_names(self):
        """The matrices of the first product, in the order of its columns: q, then k and v where the mixer has its own, then the gate."""
        s = self.spec
        return [s.q_name] + ([s.k_name, s.v_name] if s.own_kv else []) + ([s.gate] if s.gate is not None else [])

    def expected_tensors(self):
        s, p = self.spec, self.spec.prefix
        q, k, v, o = self._widths()
        rows = {s.q_name: q, s.k_name: k, s.v_name: v, s.gate: o}
        out = {p + n: ParamSpec((rows[n], s.hidden)) for n in self._in_names()}
        out[p + s.o_name] = ParamSpec((s.hidden, o))
        if s.value_blend is not None:
            out[p + s.value_blend] = ParamSpec((), init="normal")
        if s.bias:
            out.update({p + n + s.bias_suffix: ParamSpec((rows[n],), init="normal") for n in self._in_names() if n != s.gate})
            out[p + s.o_name + s.bias_suffix] = ParamSpec((s.hidden,), init="normal")
        return out

    def take_tensors(self, get):
        s, p = self.spec, self.spec.prefix
        parts = [get(p + n) for n in self._in_names()]
        rows = sum(t.shape[0] for t in parts)
        pad = (8 - rows % 8) % 8                           # rows of the product stay aligned for the attention kernels' vector loads
        if pad:
            parts.append(torch.zeros(pad, s.hidden, dtype=parts[0].dtype, device=parts[0].device))
        self.w_in = torch.cat(parts, dim=0).contiguous()
        self.w_o = get(p + s.o_name)
        if s.bias:
            like = parts[0]
            biases = [get(p + n + s.bias_suffix) if n != s.gate else torch.zeros(get(p + n).shape[0], dtype=like.dtype, device=like.device)
                      for n in self._in_names()]
            if pad:
                biases.append(torch.zeros(pad, dtype=like.dtype, device=like.device))
            self.b_in = torch.cat([b.to(like.dtype) for b in biases]).contiguous()
            self.b_o = get(p + s.o_name + s.bias_suffix)
        if s.distance_slopes is not None:
            self.slopes = torch.tensor(s.distance_slopes, dtype=torch.float32, device=self.device)
        if s.fixed_sink is not None:
            self.sink = torch.full((s.n_heads,), float(s.fixed_sink), dtype=torch.float32, device=self.device)
        if s.value_blend is not None:
            self.blend_weight = get(p + s.value_blend)

    def prepare(self, max_positions):
        from ..ops.library import for_head_dim, gated, mixers
        gated()                                            # build or load this part's kernels now, loudly
        if not self.plain_kernels:
            mixers()
            if (self.dtype == torch.bfloat16 and self.spec.head_dim == self.spec.v_head_dim
                    and kernels.attention_prefill_tcgen05_takes(self.spec.head_dim, self.spec.scale)):
                for_head_dim(self.spec.head_dim)           # prompts run on the tcgen05 kernel
        elif self.dtype == torch.bfloat16:
            for_head_dim(self.spec.head_dim)
        if isinstance(self.spec.position, RotaryPairsSpec):
            self.freq = pair_frequencies(self.spec.position, self.device)
        elif isinstance(self.spec.position, RotaryHalvesSpec):
            self.freq, self.magnitude = halves_frequencies(self.spec.position, self.device)
            if not self.spec.position.dims:
                self.freq = None

    def weights(self):
        return [t for t in (self.w_in, self.w_o, self.b_in, self.b_o, self.blend_weight) if t is not None]

    def cache_needs(self):
        s = self.spec
        if not s.own_kv:
            return CacheNeeds()
        window, keep = s.cache_span if s.cache_span is not None else (s.window, s.keep_first)
        return CacheNeeds(kv=KVNeed(s.n_kv_heads, s.head_dim, window, v_head_dim=None if s.v_head_dim == s.head_dim else s.v_head_dim,
                                    keep_first=keep if window is not None else 0))

    def gated_heads(self, h, ctx, cache_entry, owns_cache, x_norm=None):
        """The heads' outputs times the gate [T, n_heads * v_head_dim] for normed rows h (or ``x_norm`` = (stream, its norm))."""
        s = self.spec
        q_w, k_w, v_w, o_w = self._widths()
        if owns_cache != s.own_kv:
            raise ConfigError("an attention without key and value projections reads another entry's cache, one with them writes its own")
        kv = ctx.kv(cache_entry)
        if self.b_in is not None:
            proj = linear(h if h is not None else x_norm[1].forward(x_norm[0], ctx.dtype), self.w_in, self.b_in, out_dtype=ctx.dtype)
        else:
            proj = first_product(*normed_rows(h, x_norm, ctx, self.w_in), self.w_in, ctx)
        rot_dims = s.position.dims if isinstance(s.position, (RotaryPairsSpec, RotaryHalvesSpec)) else 0
        n_kv = s.n_kv_heads if s.own_kv else 0             # a row of proj then has no key and value entries
        if isinstance(s.position, RotaryHalvesSpec):
            blend_key = "value_blend:" + s.value_blend_key
            blend = None
            if s.value_blend_role == "reader":
                blend = ctx.scratch.get(blend_key)
                if blend is None:
                    raise ConfigError(f"{s.prefix}: no earlier mixer of this step has shown the values it blends with")
            kernels.rotary_half_store(proj, s.n_heads, n_kv, s.head_dim, s.v_head_dim, self.freq, rot_dims, self.magnitude, s.qk_unit_norm,
                                      s.norm_eps, ctx.tok_pos, ctx.tok_row, kv.k if owns_cache else None, kv.v if owns_cache else None,
                                      kv.table if owns_cache else None, kv.stride, blend, self.blend_weight if blend is not None else None)
            if s.value_blend_role == "source":             # this step's values, as they lie in the product's rows
                ctx.scratch[blend_key] = proj[:, q_w + k_w: q_w + k_w + v_w]
        elif rot_dims or s.qk_unit_norm or owns_cache:
            kernels.rotary_norm_store(proj, s.n_heads, n_kv, s.head_dim, s.v_head_dim, self.freq, rot_dims, s.qk_unit_norm,
                                      s.norm_eps, ctx.tok_pos, ctx.tok_row, kv.k if owns_cache else None, kv.v if owns_cache else None,
                                      kv.table if owns_cache else None, kv.stride)
        if self.plain_kernels:
            a = kernels.attention(proj, proj.shape[1], s.n_heads, s.n_kv_heads, s.head_dim, kv.k, kv.v, kv.table, kv.stride,
                                  ctx.tok_pos, ctx.tok_row, s.window, s.scale, ctx, own_rows_only=owns_cache)
        else:
            a = kernels.attention_headmix(proj, proj.shape[1], s.n_heads, s.n_kv_heads, s.head_dim, s.v_head_dim, kv.k, kv.v,
                                          kv.table, kv.stride, ctx.tok_pos, ctx.tok_row, s.window, s.scale, self.sink, None, ctx,
                                          slopes=self.slopes, keep_first=s.keep_first)
        if s.gate is None:
            return a
        return kernels.gated_norm(a, 0, None, s.norm_eps, proj, q_w + (k_w + v_w if s.own_kv else 0), "sigmoid", ctx.dtype)

    def apply(self, h, ctx, entry, cache_entry, owns_cache, out_dtype=None, x_norm=None):
        return linear(self.gated_heads(h, ctx, cache_entry, owns_cache, x_norm), self.w_o, self.b_o, out_dtype=out_dtype or ctx.dtype)

    def add_normed_to(self, x, norm, scale, ctx, entry, cache_entry, owns_cache) -> bool:
        if self.b_o is not None:
            return False                                   # the fused sum has no place for a bias
        last_product_into(x, self.gated_heads(None, ctx, cache_entry, owns_cache, (x, norm)), self.w_o, scale, ctx)
        return True
