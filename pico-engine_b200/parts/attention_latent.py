"""Softmax attention over one low-rank row per position: the cache keeps the normed latent row and one rotated key part."""
from __future__ import annotations

import torch

from ..cache import CacheNeeds, KVNeed
from ..config.specs import ConfigError, LatentAttentionSpec, RotaryHalvesSpec, RotaryPairsSpec
from ..ops import kernels, linear
from ..weights.loader import ParamSpec
from .attention_gated import halves_frequencies, pair_frequencies
from .base import Mixer, register_mixer


@register_mixer(LatentAttentionSpec)
class LatentAttention(Mixer):
    """A head's plain key is W_uk,h c for the latent row c of a position, so q_plain . k_plain = (W_uk,h^T q_plain) . c: the
    queries are carried into the latent space (a product a head, batched over the heads), and attention then reads the cached
    rows [c | rotated key part] as they are, as one key head of size rank + rot_dim whose first ``rank`` entries are also the
    value.  What comes out, sum_j p_j c_j a head, meets W_uv,h in a second batched product; the heads are multiplied by the
    sigmoid of their gate logit and projected by W_o.

    One product makes q, the down projection and the gate logits.  With ``q_rank`` that product makes the queries' own low-rank row
    instead of q; a kernel norms it (csrc/latent_ops.cu) and a second product, W_uq, makes q from it.  The rotation turns neighbours
    or halves, as the position's description says; with a window the cache gives back the pages that have left it.  The norm of the latent row, the rotation (angles from float32
    positions and float32 frequencies), the scores, the softmax and the gate are float32 in either dtype
    (csrc/latent_ops.cu, csrc/attention_headmix*.cu)."""

    takes_out_dtype = True

    def __init__(self, spec: LatentAttentionSpec, dtype, device):
        super().__init__(spec, dtype, device)
        if not isinstance(spec.position, (RotaryPairsSpec, RotaryHalvesSpec)) or spec.position.head_dim != spec.rot_dim:
            raise ConfigError("latent attention rotates pairs or halves of its rot_dim entries")
        if isinstance(spec.position, RotaryHalvesSpec) and spec.position.stretch is not None:
            raise ConfigError("latent attention takes no stretched rotation")
        if spec.window is not None and spec.window <= 0:
            raise ConfigError(f"window {spec.window} must be positive")
        if spec.position.dims > spec.rot_dim or spec.position.dims % 2:
            raise ConfigError(f"{spec.position.dims} rotated entries do not fit the rotated part of {spec.rot_dim}")
        if spec.kv_rank + spec.rot_dim > 1024:
            raise ConfigError(f"a cached row of {spec.kv_rank + spec.rot_dim} entries is not taken: up to 1024 are")
        self.state_offset = 0
        self.w_in = self.w_uk = self.w_uv = self.w_o = self.dkv_norm = self.freq = self.w_uq = self.dq_norm = None

    def _widths(self):
        """Columns of the first product: (queries, or their low-rank row; the down projection; the gate logits)."""
        s = self.spec
        q = s.n_heads * (s.head_dim + s.rot_dim) if s.q_rank is None else s.q_rank
        return q, s.kv_rank + s.rot_dim, s.n_heads if s.gate is not None else 0

    def expected_tensors(self):
        s, p = self.spec, self.spec.prefix
        q, dkv, g = self._widths()
        first = {p + s.q_name: ParamSpec((q, s.hidden))} if s.q_rank is None else \
            {p + s.dq_name: ParamSpec((q, s.hidden)), p + s.dq_norm: ParamSpec((q,), init="one_plus_normal"),
             p + s.uq_name: ParamSpec((s.n_heads * (s.head_dim + s.rot_dim), q))}
        out = {**first, p + s.dkv_name: ParamSpec((dkv, s.hidden)),
               p + s.dkv_norm: ParamSpec((s.kv_rank,), init="one_plus_normal"),
               p + s.uk_name: ParamSpec((s.n_heads * s.head_dim, s.kv_rank)), p + s.uv_name: ParamSpec((s.n_heads * s.v_head_dim, s.kv_rank)),
               p + s.o_name: ParamSpec((s.hidden, s.n_heads * s.v_head_dim))}
        if s.gate is not None:
            out[p + s.gate] = ParamSpec((g, s.hidden))
        return out

    def take_tensors(self, get):
        s, p = self.spec, self.spec.prefix
        parts = [get(p + (s.q_name if s.q_rank is None else s.dq_name)), get(p + s.dkv_name)] + ([get(p + s.gate)] if s.gate is not None else [])
        if s.q_rank is not None:
            self.w_uq, self.dq_norm = get(p + s.uq_name), get(p + s.dq_norm)
        rows = sum(t.shape[0] for t in parts)
        if rows % 8:
            parts.append(torch.zeros(8 - rows % 8, s.hidden, dtype=parts[0].dtype, device=parts[0].device))
        self.w_in = torch.cat(parts, dim=0).contiguous()
        self.w_uk = get(p + s.uk_name).view(s.n_heads, s.head_dim, s.kv_rank).contiguous()          # [H, D, rank]: q_plain @ W_uk,h
        self.w_uv = get(p + s.uv_name).view(s.n_heads, s.v_head_dim, s.kv_rank).transpose(1, 2).contiguous()   # [H, rank, Dv]
        self.w_o = get(p + s.o_name)
        self.dkv_norm = get(p + s.dkv_norm)

    def prepare(self, max_positions):
        from ..ops.library import mixers, state_space
        state_space()                                      # build or load this part's kernels now, loudly
        mixers()
        pos = self.spec.position
        if not pos.dims:
            self.freq = None
        elif isinstance(pos, RotaryHalvesSpec):
            self.freq, _ = halves_frequencies(pos, self.device)
        else:
            self.freq = pair_frequencies(pos, self.device)

    def weights(self):
        return [t for t in (self.w_in, self.w_uk, self.w_uv, self.w_o, self.dkv_norm, self.w_uq, self.dq_norm) if t is not None]

    def cache_needs(self):
        s = self.spec
        return CacheNeeds(kv=KVNeed(1, s.kv_rank + s.rot_dim, s.window, v_heads=0))

    def gated_heads(self, h, ctx, cache_entry, owns_cache):
        s = self.spec
        H, D, R, rank = s.n_heads, s.head_dim, s.rot_dim, s.kv_rank
        q_w, dkv_w, _ = self._widths()
        T = h.shape[0]
        kv = ctx.kv(cache_entry)
        proj = linear(h, self.w_in, out_dtype=ctx.dtype)
        q_rows = None
        if s.q_rank is not None:                           # the queries' own low-rank row, normed, then W_uq
            q_rows = linear(kernels.rmsnorm_cols(proj, 0, s.q_rank, self.dq_norm, s.norm_eps), self.w_uq, out_dtype=ctx.dtype)
        # the plain parts of the queries, head-major, times W_uk: [H, T, D] x [H, D, rank]
        q_plain = (proj[:, :q_w] if q_rows is None else q_rows).view(T, H, D + R)[:, :, :D].transpose(0, 1)
        # (the batched product writes a head's carried part straight into its place of the token's query row)
        q = torch.empty(T, H * (rank + R), dtype=proj.dtype, device=proj.device)
        torch.bmm(q_plain, self.w_uk, out=q.view(T, H, rank + R)[:, :, :rank].transpose(0, 1))
        kernels.latent_prepare(proj, H, D, R, rank, q_w, self.dkv_norm, s.norm_eps, self.freq, s.position.dims, None,
                               ctx.tok_pos, ctx.tok_row, kv.k if owns_cache else None, kv.table if owns_cache else None, kv.stride,
                               halves=isinstance(s.position, RotaryHalvesSpec), q_rows=q_rows, q_out=q)
        a = kernels.attention_headmix(q, q.shape[1], H, 1, rank + R, rank, kv.k, None, kv.table, kv.stride, ctx.tok_pos, ctx.tok_row,
                                      s.window, s.scale, None, None, ctx, values_in_keys=True)
        if s.gate is None:                                 # no gate: the batched product writes token-major rows itself
            out = torch.empty(T, H * s.v_head_dim, dtype=a.dtype, device=a.device)
            torch.bmm(a.view(T, H, rank).transpose(0, 1), self.w_uv, out=out.view(T, H, s.v_head_dim).transpose(0, 1))
            return out
        o = torch.bmm(a.view(T, H, rank).transpose(0, 1), self.w_uv)                        # [H, T, Dv]
        return kernels.head_gate(o, proj, q_w + dkv_w)

    def apply(self, h, ctx, entry, cache_entry, owns_cache, out_dtype=None):
        return linear(self.gated_heads(h, ctx, cache_entry, owns_cache), self.w_o, out_dtype=out_dtype or ctx.dtype)
