"""A mixture of feed-forward experts (gated or not) with a router and an optional shared expert."""
from __future__ import annotations

import torch

from ..config.specs import ConfigError, MixtureSpec
from ..ops import kernels, linear
from ..weights.loader import ParamSpec
from .base import FeedForward, first_product, last_product_into, normed_rows, register_feed_forward


@register_feed_forward(MixtureSpec)
class Mixture(FeedForward):
    """Every token uses the ``top_k`` experts with the largest router logits, weighted by the softmax over those logits;
    a shared expert runs for every token, times one sigmoid gate.  With sigmoid scores the choice reads score + a stored correction
    among the best groups of neighbouring experts, and the weights are the chosen experts' plain scores (``kernels.moe_route_grouped``).  Router and shared gate are one float32 product (their
    weights are kept in float32), the choice and the weights one kernel (csrc/gated_ops.cu: dense weights [T, experts + 1],
    zero for experts a token does not use).

    The experts run as two products on concatenated weights: gate and up of all experts (and the shared one) at once,
    then act(gate) * up * weight(token, expert) in float32, then one down product whose inner dimension runs over all
    experts' hidden units, so that the weighted sum over experts happens in the product's float32 accumulator.  Hidden
    units of experts a token does not use are exact zeros.  Every expert's weights are read in every step and every
    token multiplies with all of them: right for steps whose tokens touch most experts, n_experts / top_k times
    the necessary arithmetic for long prompts."""

    takes_out_dtype = True      # apply(..., out_dtype=) gives the product's float32 sums where the caller goes on in float32
    routes_from_stream = True   # apply(..., x_norm=(stream, norm)) lets the router read the float32 stream

    def __init__(self, spec: MixtureSpec, dtype, device):
        super().__init__(spec, dtype, device)
        if not 1 <= spec.top_k <= spec.n_experts:
            raise ConfigError(f"top_k = {spec.top_k} must lie in 1 .. n_experts = {spec.n_experts}")
        if spec.activation not in kernels.GATE_ACTIVATIONS:
            raise ConfigError(f"activation {spec.activation!r} is not known")
        if spec.scores not in ("softmax_chosen", "softmax_all", "sigmoid"):
            raise ConfigError(f"scores must be \"softmax_chosen\", \"softmax_all\" or \"sigmoid\", not {spec.scores!r}")
        if spec.scores == "sigmoid":
            if spec.shared_intermediate is not None:
                raise ConfigError("sigmoid scores come without a shared expert")
            per = spec.n_experts // max(spec.n_groups, 1)
            if (spec.n_groups < 1 or spec.n_experts % spec.n_groups or not 1 <= spec.keep_groups <= spec.n_groups
                    or spec.keep_groups * per < spec.top_k or spec.group_best < 1):
                raise ConfigError(f"{spec.n_experts} experts in {spec.n_groups} groups of which {spec.keep_groups} stay cannot give {spec.top_k}")
        elif spec.correction_name is not None or spec.n_groups != 1:
            raise ConfigError("a correction and groups of experts belong to sigmoid scores")
        self.w_router = self.w_gate_up = self.w_down = self.correction = None

    def _experts(self):
        s = self.spec
        names = [(s.prefix + s.expert_name.format(e) + ".", s.intermediate) for e in range(s.n_experts)]
        if s.shared_intermediate is not None:
            names.append((s.prefix + s.shared_name + ".", s.shared_intermediate))
        return names

    def _shared_gate(self) -> bool:
        return self.spec.shared_intermediate is not None and self.spec.shared_gate_name is not None

    def _extra(self):
        """What the routing kernels make of the column behind the experts': nothing, sigmoid(gate logit), or 1."""
        return False if self.spec.shared_intermediate is None else (True if self._shared_gate() else "one")

    def expected_tensors(self):
        s = self.spec
        out = {s.prefix + s.router_name: ParamSpec((s.n_experts, s.hidden))}
        for p, ff in self._experts():
            if s.gated:
                out[p + s.gate_name] = ParamSpec((ff, s.hidden))
            out.update({p + s.up_name: ParamSpec((ff, s.hidden)), p + s.down_name: ParamSpec((s.hidden, ff))})
        if self._shared_gate():
            out[s.prefix + s.shared_gate_name] = ParamSpec((1, s.hidden))
        if s.correction_name is not None:
            out[s.prefix + s.correction_name] = ParamSpec((s.n_experts,))
        return out

    def take_tensors(self, get):
        s = self.spec
        router = [get(s.prefix + s.router_name)] + ([get(s.prefix + s.shared_gate_name)] if self._shared_gate() else [])
        self.w_router = torch.cat(router, dim=0).float().contiguous()           # router logits are float32 products
        experts = self._experts()
        gates = [get(p + s.gate_name) for p, _ in experts] if s.gated else []
        self.w_gate_up = torch.cat(gates + [get(p + s.up_name) for p, _ in experts], dim=0).contiguous()
        self.w_down = torch.cat([get(p + s.down_name) for p, _ in experts], dim=1).contiguous()
        if s.correction_name is not None:
            self.correction = get(s.prefix + s.correction_name).float().contiguous()

    def prepare(self, max_positions):
        from ..ops.library import gated
        gated()                                            # build or load this part's kernels now, loudly

    def routing(self, h):
        """Dense weights float32 [T, n_experts (+ 1)] of rows h."""
        s = self.spec
        logits = linear(h, self.w_router, out_dtype=torch.float32)
        if s.scores == "sigmoid":
            return kernels.moe_route_grouped(logits, s.n_experts, s.top_k, self.correction, s.n_groups, s.keep_groups, s.group_best,
                                             s.route_scale)
        return kernels.moe_route(logits, s.n_experts, s.top_k, self._extra(), over_all=s.scores == "softmax_all", factor=s.route_scale)

    def _activation(self, h, ctx, x_norm=None):
        s = self.spec
        from .block import PassThrough
        from .norm import RMSNorm
        how = {"over_all": s.scores == "softmax_all", "factor": s.route_scale}
        if (x_norm is not None and type(x_norm[1]) in (RMSNorm, PassThrough) and s.n_experts <= kernels.MOE_ROUTE_STREAM_MAX_EXPERTS
                and s.scores != "sigmoid"):
            # the router reads the float32 stream itself (its norm, where it has one, is part of the routing kernel): the same
            # logits however the step is cut, and the gate/up product may take the norm into its prologue
            x, norm = x_norm
            if type(norm) is RMSNorm:
                weights = kernels.moe_route_stream(x, norm.weight, norm.eps, self.w_router, s.n_experts, s.top_k, self._extra(), **how)
                gate_up = first_product(*normed_rows(None, x_norm, ctx, self.w_gate_up), self.w_gate_up, ctx)
            else:
                weights = kernels.moe_route_stream(x, None, 0.0, self.w_router, s.n_experts, s.top_k, self._extra(), **how)
                gate_up = linear(norm.forward(x, ctx.dtype) if h is None else h, self.w_gate_up, out_dtype=ctx.dtype)
        else:
            from .norm import LayerNorm
            if h is None:
                h = x_norm[1].forward(x_norm[0], ctx.dtype)
            if (x_norm is not None and s.scores == "sigmoid" and type(x_norm[1]) is LayerNorm
                    and s.n_experts <= kernels.MOE_ROUTE_STREAM_MAX_EXPERTS):
                # the router reads the float32 stream through its layer norm inside the routing kernel
                x, norm = x_norm
                weights = kernels.moe_route_stream_grouped(x, norm.weight, norm.bias, norm.eps, self.w_router, s.n_experts, s.top_k,
                                                           self.correction, s.n_groups, s.keep_groups, s.group_best, s.route_scale)
            else:
                weights = self.routing(h)
            gate_up = linear(h, self.w_gate_up, out_dtype=ctx.dtype)
        if not s.gated:
            return kernels.weighted_act(gate_up, s.activation, weights, s.intermediate)
        return kernels.gated_act(gate_up, s.activation, weights, s.intermediate)

    def apply(self, h, ctx, out_dtype=None, x_norm=None):
        """``x_norm`` = (float32 stream, its norm or pass-through): the router then reads the stream itself."""
        return linear(self._activation(h, ctx, x_norm), self.w_down, out_dtype=out_dtype or ctx.dtype)

    def add_normed_to(self, x, norm, scale, ctx) -> bool:
        """x += scale * mixture(norm(x)); the sum is the last product's epilogue where it takes the sizes."""
        last_product_into(x, self._activation(None, ctx, (x, norm)), self.w_down, scale, ctx)
        return True
