"""A layer: the parts it has (a mixer, a feed-forward, a norm before each; any of them may be
absent) and the arrangement that runs them around the residual stream."""
from __future__ import annotations

from ..config.specs import ConfigError, LayerSpec
from ..cache import CacheNeeds
from ..weights.loader import ParamSpec
from .base import ARRANGEMENTS, FEED_FORWARDS, INPUT_FILTERS, MIXERS, NORMS, Norm, Part, build_part, register_arrangement


class PassThrough(Norm):
    """Stands where a half of a block has no norm: the residual stream as it is, in the step's dtype."""

    def __init__(self, dtype, device):
        super().__init__(None, dtype, device)

    def forward(self, x, out_dtype, rows_index=None):
        rows = x if rows_index is None else x.index_select(0, rows_index.long())
        return rows.to(out_dtype)


class ScaleVector(Part):
    """A learned vector [hidden] that a sublayer's normed output is multiplied by before it is added to the stream."""

    def __init__(self, name: str, size: int, dtype, device):
        super().__init__(None, dtype, device)
        self.name, self.size, self.vector = name, size, None
        self.folded = {}

    def expected_tensors(self):
        return {self.name: ParamSpec((self.size,), init="one_plus_normal")}

    def take_tensors(self, get):
        self.vector = get(self.name)

    def weights(self):
        return [self.vector]

    def times(self, norm_weight):
        """norm weight * this vector, element by element, formed once in float32."""
        key = norm_weight.data_ptr()
        if key not in self.folded:
            self.folded[key] = (norm_weight.float() * self.vector.float()).contiguous()
        return self.folded[key]


def _hidden_of(spec: LayerSpec) -> int:
    for part in (spec.mixer_norm, spec.feed_forward_norm, spec.mixer, spec.feed_forward):
        for field in ("size", "hidden"):
            if part is not None and hasattr(part, field):
                return getattr(part, field)
    raise ConfigError("a scaled sublayer output needs a part that knows the stream's width")


class Layer:
    def __init__(self, spec: LayerSpec, dtype, device):
        self.spec = spec
        if spec.mixer is None and spec.feed_forward is None:
            raise ConfigError("a layer needs a mixer or a feed-forward")

        def build(table, kind, part_spec):
            return None if part_spec is None else build_part(table, kind, part_spec, dtype, device)
        self.mixer = build(MIXERS, "mixer", spec.mixer)
        self.feed_forward = build(FEED_FORWARDS, "feed-forward", spec.feed_forward)
        self.mixer_norm = build(NORMS, "norm", spec.mixer_norm) or PassThrough(dtype, device)
        self.feed_forward_norm = build(NORMS, "norm", spec.feed_forward_norm) or PassThrough(dtype, device)
        self.mixer_input = build(INPUT_FILTERS, "input filter", spec.mixer_input)
        self.feed_forward_input = build(INPUT_FILTERS, "input filter", spec.feed_forward_input)
        self.mixer_out_norm = build(NORMS, "norm", spec.mixer_out_norm)
        self.feed_forward_out_norm = build(NORMS, "norm", spec.feed_forward_out_norm)
        self.mixer_scale = None if spec.mixer_scale is None else ScaleVector(spec.mixer_scale, _hidden_of(spec), dtype, device)
        self.feed_forward_scale = None if spec.feed_forward_scale is None else \
            ScaleVector(spec.feed_forward_scale, _hidden_of(spec), dtype, device)
        if (self.mixer_input is not None and self.mixer is None) or (self.feed_forward_input is not None and self.feed_forward is None):
            raise ConfigError("an input filter needs the sublayer whose input it filters")
        try:
            self._run = ARRANGEMENTS[spec.arrangement]
        except KeyError:
            raise ConfigError(f"unknown arrangement {spec.arrangement!r}; known: {', '.join(sorted(ARRANGEMENTS))}") from None

    def parts(self):
        """The parts that are there (a stand-in for an absent norm has no tensors and is left out)."""
        return tuple(p for p in (self.mixer, self.mixer_norm, self.mixer_input, self.feed_forward, self.feed_forward_norm,
                                 self.feed_forward_input, self.mixer_scale, self.feed_forward_scale, self.mixer_out_norm,
                                 self.feed_forward_out_norm)
                     if p is not None and not isinstance(p, PassThrough))

    def cache_needs(self):
        """What one execution of the layer keeps in the cache: the mixer's keys, values and state, and behind the
        mixer's state the states of the input filters (``state_offsets``).  None: nothing."""
        mixer = self.mixer.cache_needs() if self.mixer is not None else CacheNeeds()
        extra = sum(f.state_elems() for f in (self.mixer_input, self.feed_forward_input) if f is not None)
        if not extra:
            return mixer if self.mixer is not None else None
        if mixer.state_elems and mixer.state_dtype != "float32":
            raise ConfigError("input filters keep float32 state; a mixer beside them must keep float32 state too")
        return CacheNeeds(kv=mixer.kv, state_elems=mixer.state_elems + extra, state_dtype="float32")

    def state_offsets(self):
        """(offset of the mixer input filter's state, offset of the feed-forward input filter's) in a slot's row."""
        first = self.mixer.cache_needs().state_elems if self.mixer is not None else 0
        return first, first + (self.mixer_input.state_elems() if self.mixer_input is not None else 0)

    def run(self, x, ctx, entry: int, cache_entry: int, owns_cache: bool) -> None:
        self._run(self, x, ctx, entry, cache_entry, owns_cache)


@register_arrangement("pre_norm")
def pre_norm(layer: Layer, x, ctx, entry, cache_entry, owns_cache) -> None:
    """x += mixer(norm(x)); x += feed_forward(norm(x))  (pico-engine src/pico_engine/model.py:167-237).  With a
    ``residual_scale`` m other than 1 both sums are x += m * sublayer(norm(x)), formed in float32 from the sublayer's
    output (a part may do the sum itself: ``add_scaled_to``)."""
    m = getattr(getattr(layer, "spec", None), "residual_scale", 1.0)
    if m != 1.0:
        from ..ops import kernels
        ctx.settle(x)
        halves = ((layer.mixer, layer.mixer_norm, (entry, cache_entry, owns_cache)), (layer.feed_forward, layer.feed_forward_norm, ()))
        for part, norm, where in halves:
            if part is None:
                continue
            # a part may do the whole half itself (the norm in the prologue of its first product, the scaled sum in the
            # epilogue of its last one, for steps of few rows); it says whether it did
            fused = getattr(part, "add_normed_to", None)
            if fused is not None and fused(x, norm, m, ctx, *where):
                continue
            h = norm.forward(x, ctx.dtype)
            if hasattr(part, "add_scaled_to"):
                part.add_scaled_to(x, h, m, ctx, *where)
            else:
                wide = {"out_dtype": x.dtype} if getattr(part, "takes_out_dtype", False) else {}
                kernels.scaled_add(x, part.apply(h, ctx, *where, **wide).contiguous(), m)
        return
    if layer.mixer is not None:
        if not layer.mixer.takes_pending:
            ctx.settle(x)
        layer.mixer.add_to(x, layer.mixer_norm, ctx, entry, cache_entry, owns_cache)
    if layer.feed_forward is not None:
        if not layer.feed_forward.takes_pending:
            ctx.settle(x)
        layer.feed_forward.add_to(x, layer.feed_forward_norm, ctx)


@register_arrangement("parallel")
def parallel(layer: Layer, x, ctx, entry, cache_entry, owns_cache) -> None:
    """x += mixer(f1(norm1(x))) + feed_forward(f2(norm2(x))): both halves read the same x (f1, f2: the input filters,
    where the layer has them).  Both inputs are made before either half adds its output to the stream.  Layer norms
    followed by convolutions of equal taps are one kernel for both halves, which reads the stream once."""
    from ..ops import kernels
    from .input_conv import CausalConvAdd
    from .norm import LayerNorm
    ctx.settle(x)
    halves = [(layer.mixer, layer.mixer_norm, layer.mixer_input), (layer.feed_forward, layer.feed_forward_norm, layer.feed_forward_input)]
    offsets = layer.state_offsets()
    live = [(part, norm, filt, off) for (part, norm, filt), off in zip(halves, offsets) if part is not None]
    state = ctx.state(cache_entry) if any(f is not None and f.state_elems() for _, _, f, _ in live) else None
    fusable = (all(type(n) is LayerNorm and type(f) is CausalConvAdd for _, n, f, _ in live)
               and len({(n.eps, f.spec.taps) for _, n, f, _ in live}) == 1
               and live[0][2].spec.taps <= kernels.DUAL_NORM_CONV_MAX_TAPS)
    if fusable:
        if state is None:                                  # one tap: nothing is kept, the kernel is handed any float32 row
            state = ctx.scratch.setdefault("no_state", x.new_zeros(1, 1))
        inputs = kernels.dual_layernorm_conv(x, [(n.weight, n.bias, f.taps_weight, off) for _, n, f, off in live], live[0][1].eps,
                                             state, ctx.tok_row, ctx.row_first, ctx.row_lens, ctx.slots, ctx.dtype, ctx.one_token_each)
    else:
        inputs = []
        for _, norm, filt, off in live:
            inputs.append(norm.forward(x, ctx.dtype) if filt is None
                          else filt.apply(norm.forward(x, x.dtype), ctx, state, off, ctx.dtype))
    for (part, _, _, _), h in zip(live, inputs):
        if part is layer.mixer:
            if hasattr(part, "add_output_to"):
                part.add_output_to(x, h, ctx, entry, cache_entry, owns_cache)
            else:
                kernels.residual_add(x, part.apply(h, ctx, entry, cache_entry, owns_cache).contiguous())
        elif hasattr(part, "add_output_to"):
            part.add_output_to(x, h, ctx)
        else:
            kernels.residual_add(x, part.apply(h, ctx).contiguous())


@register_arrangement("post_norm")
def post_norm(layer: Layer, x, ctx, entry, cache_entry, owns_cache) -> None:
    """x += s1 * norm1(mixer(x)); x += s2 * norm2(feed_forward(x)): the sublayers read the stream as it is (rounded to the
    step's dtype where that is not float32), the norms act on their outputs, s1 and s2 are learned vectors (absent: ones).
    A sublayer hands over the float32 sums of its last product; norm, scale and the sum into the stream are one kernel in
    float32.  A feed-forward that routes is also handed the float32 stream, so that its router reads that."""
    from ..ops import kernels
    from .norm import RMSNorm
    ctx.settle(x)
    halves = ((layer.mixer, layer.mixer_norm, layer.mixer_scale, (entry, cache_entry, owns_cache)),
              (layer.feed_forward, layer.feed_forward_norm, layer.feed_forward_scale, ()))
    reads = PassThrough(ctx.dtype, x.device)
    for part, norm, scale, where in halves:
        if part is None:
            continue
        if type(norm) is not RMSNorm:
            raise ConfigError("the post_norm arrangement takes an RMS norm on every sublayer's output")
        h = reads.forward(x, ctx.dtype)
        extra = {"out_dtype": x.dtype} if getattr(part, "takes_out_dtype", False) else {}
        if part is layer.feed_forward and getattr(part, "routes_from_stream", False):
            extra["x_norm"] = (x, reads)
        y = part.apply(h, ctx, *where, **extra)
        if y.dtype != x.dtype:
            y = y.float()
        kernels.normed_sum_add(x, [y.contiguous()], [norm.weight.float().contiguous() if scale is None else scale.times(norm.weight)],
                               norm.eps, 1.0)


@register_arrangement("sandwich")
def sandwich(layer: Layer, x, ctx, entry, cache_entry, owns_cache) -> None:
    """x += out_norm1(mixer(norm1(x))); x += out_norm2(feed_forward(norm2(x))): a norm before and one after each sublayer.  A
    sublayer hands over the float32 sums of its last product where it can; its output norm and the sum into the stream are left
    pending, so that they and the norm in front of whatever reads the stream next are one kernel in float32."""
    halves = ((layer.mixer, layer.mixer_norm, layer.mixer_out_norm, (entry, cache_entry, owns_cache)),
              (layer.feed_forward, layer.feed_forward_norm, layer.feed_forward_out_norm, ()))
    for part, norm, out_norm, where in halves:
        if part is None:
            continue
        if out_norm is None:
            raise ConfigError("the sandwich arrangement takes a norm on every sublayer's output")
        h = ctx.normed(x, norm)
        extra = {"out_dtype": x.dtype} if getattr(part, "takes_out_dtype", False) else {}
        if part is layer.feed_forward and getattr(part, "routes_from_stream", False):
            extra["x_norm"] = (x, norm)                      # a router may read the float32 stream through the norm itself
        ctx.defer_normed_add(x, part.apply(h, ctx, *where, **extra), out_norm)
