"""Dense feed-forwards: gated (SwiGLU) and plain (up, activation, down)."""
from __future__ import annotations

import torch

from ..config.specs import ConfigError, DenseMLPSpec, GatedMLPSpec, SwiGLUSpec
from ..ops import kernels, linear
from ..weights.loader import ParamSpec
from .base import FeedForward, first_product, last_product_into, normed_rows, register_feed_forward


@register_feed_forward(SwiGLUSpec)
class SwiGLU(FeedForward):
    """down(silu(gate(h)) * up(h)) with gate and up as one product on concatenated weights
    (pico-engine src/pico_engine/model.py:95-98, 222-235; kernels.py:62-74)."""

    def __init__(self, spec: SwiGLUSpec, dtype, device):
        super().__init__(spec, dtype, device)
        self.w_gate_up = self.w_down = None

    def expected_tensors(self):
        s = self.spec
        return {s.prefix + s.gate_name + ".weight": ParamSpec((s.intermediate, s.hidden)),
                s.prefix + s.up_name + ".weight": ParamSpec((s.intermediate, s.hidden)),
                s.prefix + s.down_name + ".weight": ParamSpec((s.hidden, s.intermediate))}

    def take_tensors(self, get):
        s = self.spec
        self.w_gate_up = torch.cat([get(s.prefix + s.gate_name + ".weight"),
                                    get(s.prefix + s.up_name + ".weight")], dim=0).contiguous()
        self.w_down = get(s.prefix + s.down_name + ".weight")

    def _activation(self, h, ctx):
        from ..ops.linear import gate_up_swiglu
        return gate_up_swiglu(h, self.w_gate_up)

    def apply(self, h, ctx):
        return linear(self._activation(h, ctx), self.w_down, out_dtype=ctx.dtype)

    takes_pending = True

    def add_to(self, x, norm, ctx):
        from .norm import RMSNorm
        if (ctx.dtype == torch.bfloat16 and type(norm) is RMSNorm and self.spec.intermediate % 8 == 0
                and kernels.decode_fused_takes(x.shape[0], self.w_gate_up, x) and kernels.decode_fused_takes(x.shape[0], self.w_down)):
            # decoding a few sequences: norm, gate and up products and the activation are one kernel
            ctx.settle(x)
            act = kernels.norm_gate_up_swiglu(x, norm.weight, norm.eps, self.w_gate_up)
            kernels.linear_fused(act, self.w_down, accumulate_into=x)
            return
        linear(self._activation(ctx.normed(x, norm), ctx), self.w_down, accumulate_into=x,
               defer_add=lambda y: ctx.defer_add(x, y))


@register_feed_forward(DenseMLPSpec)
class DenseMLP(FeedForward):
    """down(act(up(h))) without biases; act is the square of relu, gelu (tanh formula) or silu, computed in float32."""

    def __init__(self, spec: DenseMLPSpec, dtype, device):
        super().__init__(spec, dtype, device)
        if spec.activation not in kernels.ACTIVATIONS:
            raise ConfigError(f"activation {spec.activation!r} is not known; known: {', '.join(sorted(kernels.ACTIVATIONS))}")
        self.w_up = self.w_down = None

    def expected_tensors(self):
        s = self.spec
        return {s.prefix + s.up_name: ParamSpec((s.intermediate, s.hidden)),
                s.prefix + s.down_name: ParamSpec((s.hidden, s.intermediate))}

    def take_tensors(self, get):
        s = self.spec
        self.w_up, self.w_down = get(s.prefix + s.up_name), get(s.prefix + s.down_name)

    def _activation(self, h, ctx):
        up = linear(h, self.w_up, out_dtype=ctx.dtype)
        return kernels.activation(up, self.spec.activation, out=up)

    def apply(self, h, ctx):
        return linear(self._activation(h, ctx), self.w_down, out_dtype=ctx.dtype)

    def add_output_to(self, x, h, ctx) -> None:
        """x += feed_forward(h) for rows h that are normed (and filtered) already."""
        linear(self._activation(h, ctx), self.w_down, accumulate_into=x)


@register_feed_forward(GatedMLPSpec)
class GatedMLP(FeedForward):
    """down(act(gate(h)) * up(h)) without biases, gate and up as one product on concatenated weights; act is gelu
    (tanh formula) or silu, or the clamped form min(gate, l) sigmoid(a min(gate, l)) (clamp(up, -l, l) + 1); formed in float32."""

    takes_out_dtype = True      # apply(..., out_dtype=) gives the product's float32 sums where the caller goes on in float32

    def __init__(self, spec: GatedMLPSpec, dtype, device):
        super().__init__(spec, dtype, device)
        if spec.activation not in ("gelu_tanh", "silu", "clamped_sigmoid"):
            raise ConfigError(f"activation {spec.activation!r} is not known; known: gelu_tanh, silu, clamped_sigmoid")
        if spec.activation == "clamped_sigmoid" and not (spec.limit is not None and spec.limit > 0):
            raise ConfigError(f"the clamped activation needs a positive limit, found {spec.limit!r}")
        self.w_gate_up = self.w_down = None

    def expected_tensors(self):
        s = self.spec
        return {s.prefix + s.gate_name: ParamSpec((s.intermediate, s.hidden)), s.prefix + s.up_name: ParamSpec((s.intermediate, s.hidden)),
                s.prefix + s.down_name: ParamSpec((s.hidden, s.intermediate))}

    def take_tensors(self, get):
        s = self.spec
        self.w_gate_up = torch.cat([get(s.prefix + s.gate_name), get(s.prefix + s.up_name)], dim=0).contiguous()
        self.w_down = get(s.prefix + s.down_name)

    def prepare(self, max_positions):
        from ..ops.library import gated
        gated()                                            # build or load this part's kernels now, loudly

    def _activation(self, h, ctx, x_norm=None):
        if self.spec.activation == "silu" and x_norm is None:
            from ..ops.linear import gate_up_swiglu
            return gate_up_swiglu(h, self.w_gate_up)
        gate_up = first_product(*normed_rows(h, x_norm, ctx, self.w_gate_up), self.w_gate_up, ctx)
        return kernels.gated_act(gate_up, self.spec.activation, limit=self.spec.limit or 0.0, alpha=self.spec.alpha)

    def apply(self, h, ctx, out_dtype=None):
        return linear(self._activation(h, ctx), self.w_down, out_dtype=out_dtype or ctx.dtype)

    def add_normed_to(self, x, norm, scale, ctx) -> bool:
        """x += scale * feed_forward(norm(x)), the norm in the first product and the sum in the last where they take the sizes."""
        last_product_into(x, self._activation(None, ctx, (x, norm)), self.w_down, scale, ctx)
        return True
