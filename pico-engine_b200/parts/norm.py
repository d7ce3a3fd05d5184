"""RMSNorm and layer norm."""
from __future__ import annotations

from ..config.specs import LayerNormSpec, RMSNormSpec
from ..ops import kernels
from ..weights.loader import ParamSpec
from .base import Norm, register_norm


@register_norm(RMSNormSpec)
class RMSNorm(Norm):
    """y = x * rsqrt(mean(x^2) + eps) * w in float32 (pico-engine src/pico_engine/kernels.py:14-23).
    The weight stays in the dtype it was stored in; with ``one_plus`` the stored vector v lies around zero, w = 1 + v is
    formed once in float32 and kept so."""

    def __init__(self, spec: RMSNormSpec, dtype, device):
        super().__init__(spec, dtype, device)
        self.weight = None
        self.eps = spec.eps

    def expected_tensors(self):
        return {self.spec.weight: ParamSpec((self.spec.size,), init="normal" if self.spec.one_plus else "one_plus_normal")}

    def take_tensors(self, get):
        self.weight = get(self.spec.weight)
        if self.spec.one_plus:
            self.weight = (1.0 + self.weight.float()).contiguous()

    def forward(self, x, out_dtype, rows_index=None):
        return kernels.rmsnorm(x, self.weight, self.eps, out_dtype, rows_index)

    def add_forward(self, x, y, out_dtype):
        return kernels.add_rmsnorm(x, y, self.weight, self.eps, out_dtype)


@register_norm(LayerNormSpec)
class LayerNorm(Norm):
    """y = (x - mean) / sqrt(var + eps) * w + b in float32, var the mean of the squared deviations."""

    def __init__(self, spec: LayerNormSpec, dtype, device):
        super().__init__(spec, dtype, device)
        self.weight = self.bias = None
        self.eps = spec.eps

    def expected_tensors(self):
        return {self.spec.weight: ParamSpec((self.spec.size,), init="one_plus_normal"),
                self.spec.bias: ParamSpec((self.spec.size,))}

    def take_tensors(self, get):
        self.weight, self.bias = get(self.spec.weight), get(self.spec.bias)

    def prepare(self, max_positions):
        from ..ops.library import mixers
        mixers()                                           # build or load this part's kernels now, loudly

    def forward(self, x, out_dtype, rows_index=None):
        return kernels.layernorm(x, self.weight, self.bias, self.eps, out_dtype, rows_index)

    def add_into(self, x, y, then=None, out_dtype=None):
        """x += layernorm(y); with a layer norm ``then`` its rows of the new x come out of the same kernel."""
        if then is None:
            return kernels.layernorm_add(x, y, self.weight, self.bias, self.eps)
        if type(then) is LayerNorm:
            return kernels.layernorm_add(x, y, self.weight, self.bias, self.eps, (then.weight, then.bias, then.eps), out_dtype)
        kernels.layernorm_add(x, y, self.weight, self.bias, self.eps)
        return then.forward(x, out_dtype)
