"""A selective state-space mixer with a scalar decay a head: short convolution, recurrence over a matrix state, gate, norm."""
from __future__ import annotations

import torch

from ..cache import CacheNeeds
from ..config.specs import ConfigError, StateSpaceSpec
from ..ops import kernels, linear
from ..weights.loader import ParamSpec
from .base import Mixer, register_mixer


@register_mixer(StateSpaceSpec)
class StateSpace(Mixer):
    """One product makes z | x | B | C | dt.  x, B and C pass the causal convolution and silu (float32 out); the recurrence
    S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T, y_t = S_t^T C_t + D x_t runs in float32 with its state in the layer's
    row of the cache's state area; y * silu(z) is normed in equal runs of channels and projected by W_o
    (csrc/state_space.cu).  A sequence's row of the state area holds the matrix states (in the recurrence kernel's own order)
    and behind them the convolution's last ``taps`` - 1 inputs, both float32, both zero when a sequence starts.  All that is
    read of the step lies on the device, so a decode step can be a captured graph."""

    takes_out_dtype = True

    def __init__(self, spec: StateSpaceSpec, dtype, device):
        super().__init__(spec, dtype, device)
        if spec.n_heads % spec.n_groups:
            raise ConfigError(f"{spec.n_heads} heads cannot share {spec.n_groups} groups evenly")
        if (spec.n_heads * spec.head_dim) % spec.norm_groups:
            raise ConfigError(f"{spec.norm_groups} norm groups do not divide {spec.n_heads * spec.head_dim} channels")
        if spec.state > 512 or spec.taps < 1:
            raise ConfigError(f"state size {spec.state} / {spec.taps} taps are not taken: up to 512 state rows, at least one tap")
        self.state_offset = 0
        self.w_in = self.w_o = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.d_skip = self.norm = None
        self._state_elems = None

    def _sizes(self):
        s = self.spec
        inner, bc = s.n_heads * s.head_dim, s.n_groups * s.state
        return inner, bc, inner + 2 * bc                       # z or x; B or C; the convolved channels

    def expected_tensors(self):
        s, p = self.spec, self.spec.prefix
        inner, bc, conv = self._sizes()
        return {p + s.in_name: ParamSpec((2 * inner + 2 * bc + s.n_heads, s.hidden)),
                p + s.conv_name: ParamSpec((conv, s.taps)), p + s.conv_name + s.bias_suffix: ParamSpec((conv,)),
                p + s.dt_bias_name: ParamSpec((s.n_heads,)), p + s.a_log_name: ParamSpec((s.n_heads,)),
                p + s.d_name: ParamSpec((s.n_heads,), init="one_plus_normal"),
                p + s.norm_name: ParamSpec((inner,), init="one_plus_normal"), p + s.o_name: ParamSpec((s.hidden, inner))}

    def take_tensors(self, get):
        s, p = self.spec, self.spec.prefix
        self.w_in, self.w_o = get(p + s.in_name), get(p + s.o_name)
        self.conv_w, self.conv_b = get(p + s.conv_name), get(p + s.conv_name + s.bias_suffix)
        # what enters the recurrence is float32
        self.dt_bias, self.a_log, self.d_skip = (get(p + n).float().contiguous() for n in (s.dt_bias_name, s.a_log_name, s.d_name))
        self.norm = get(p + s.norm_name)

    def prepare(self, max_positions):
        from ..ops.library import state_space
        state_space()                                      # build or load this part's kernels now, loudly

    def weights(self):
        return [self.w_in, self.w_o, self.conv_w, self.conv_b, self.dt_bias, self.a_log, self.d_skip, self.norm]

    def matrix_state_elems(self) -> int:
        if self._state_elems is None:
            s = self.spec
            self._state_elems = kernels.state_space_elems(s.n_heads, s.head_dim, s.state)
        return self._state_elems

    def cache_needs(self):
        s = self.spec
        return CacheNeeds(kv=None, state_elems=self.matrix_state_elems() + (s.taps - 1) * self._sizes()[2])

    def chunks_pay(self, lens) -> bool:
        """Whether a step with these numbers of tokens a row runs its recurrence in chunks.  One walk a sequence takes as long as
        the longest row, however empty that leaves the GPU; in chunks of 64 every token is walked twice, but all chunks run side
        by side.  Both are counted in token times a wave of blocks (about two blocks of 256 threads an SM on 148 SMs), the
        carry pass as one chunk more.  Either way gives the same numbers up to float32 rounding."""
        longest = max(lens, default=0)
        if longest <= 64:
            return False
        s = self.spec
        split = kernels.state_space_split(s.state)
        per = s.n_heads * -(-s.head_dim // min(s.head_dim, 256 // split))     # blocks a sequence or chunk
        wave = 296
        walk = longest * -(-sum(1 for n in lens if n > 0) * per // wave)
        chunks = sum(-(-n // 64) for n in lens)
        return 64 * (2 * -(-chunks * per // wave) + 1) < walk

    def normed_output(self, h, ctx, cache_entry):
        s = self.spec
        inner, bc, conv = self._sizes()
        state = ctx.state(cache_entry)
        proj = linear(h, self.w_in, out_dtype=ctx.dtype)
        xbc = kernels.conv_silu(proj, inner, conv, self.conv_w, self.conv_b, state, self.state_offset + self.matrix_state_elems(),
                                ctx.tok_row, ctx.row_first, ctx.row_lens, ctx.slots)
        y = kernels.state_space_scan(xbc, proj, inner + conv, self.dt_bias, self.a_log, self.d_skip, state, self.state_offset,
                                     ctx.row_first, ctx.row_lens, ctx.slots, s.n_heads, s.head_dim, s.state, s.n_groups,
                                     chunked=self.chunks_pay(ctx.lens))
        return kernels.gate_norm(y, inner // s.norm_groups, proj, 0, self.norm, s.norm_eps)

    def apply(self, h, ctx, entry, cache_entry, owns_cache, out_dtype=None):
        return linear(self.normed_output(h, ctx, cache_entry), self.w_o, out_dtype=out_dtype or ctx.dtype)
