"""RMSNorm, alone or fused with the residual sum.

ullm/layers/layernorm.py:20-34: everything in 32-bit; with a residual the sum
x + residual is normed unrounded and its rounded value becomes the new
residual; the weight multiplies before the cast back.
"""

from __future__ import annotations

from ..csrc import kernels
from .base import Norm, ParamDecl
from .registry import register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, size: int, eps: float, param: str = "weight"):
        """`param`: the name of the weight behind the norm's prefix (may be empty: the prefix is the name)."""
        super().__init__()
        self.size = size
        self.eps = eps
        self.param = param

    def param_decls(self):
        return {self.param: ParamDecl((self.size,), "norm")}

    @property
    def weight(self):
        return self.tensors[self.param]

    def rms_params(self):
        return self.weight, self.eps

    def row_params(self):
        return self.weight, self.eps, False

    def scale_add(self, a, stream, mult: float, copy=None):
        kernels().norm_scale_add(a, stream, self.weight, self.eps, mult, copy)
        return stream

    def forward_rows(self, stream, rows, out):
        kernels().rmsnorm_rows_f32(stream, rows, self.weight, self.eps, out)
        return out

    def forward(self, x, residual=None, out=None):
        """x [T, size].  residual (same shape), if given, is updated in place
        to x + residual.  Returns the normed rows (in `out` if given; `out`
        may be `x`)."""
        if out is None:
            out = x
        kernels().add_rmsnorm(x, residual, self.weight, self.eps, out)
        return out


@register_norm("layernorm")
class LayerNorm(Norm):
    """(x - mean) / sqrt(variance + eps) * weight over the row, the variance being the mean of the squared
    deviations; a weight and no bias.  It reads and writes a 32-bit residual stream (`forward_rows`, `scale_add`)
    or norms plain rows (`forward`); sums are 32-bit, one rounding at the store."""

    def __init__(self, size: int, eps: float, param: str = "weight"):
        super().__init__()
        self.size = size
        self.eps = eps
        self.param = param

    def param_decls(self):
        return {self.param: ParamDecl((self.size,), "norm")}

    @property
    def weight(self):
        return self.tensors[self.param]

    def row_params(self):
        return self.weight, self.eps, True

    def scale_add(self, a, stream, mult: float, copy=None):
        if copy is not None:
            raise NotImplementedError("a rounded copy of the stream beside a centred norm")
        kernels().norm_add_norm(stream, a, self.weight, self.eps, mult, center=True)
        return stream

    def forward_rows(self, stream, rows, out):
        kernels().norm_rows(stream, rows, self.weight, self.eps, out, center=True)
        return out
