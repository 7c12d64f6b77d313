"""Gated feed-forward: down(act(gate(x)) * up(x)), gate and up as one matrix
with rows gate | up (ullm/models/qwen3.py:23-46, ullm/layers/linear.py:490-491,
ullm/layers/activation.py:16-18)."""

from __future__ import annotations

from ..csrc import kernels
from .base import FeedForward, ParamDecl
from .linear import linear
from .registry import register_feed_forward

_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}
# "swiglu_clamped": g' = min(gate, limit), u' = clamp(up, -limit, limit), g' * sigmoid(alpha g') * (u' + 1)
_CLAMPED = "swiglu_clamped"


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu", limit: float | None = None,
                 alpha: float = 1.702, names: dict | None = None):
        """`limit`, `alpha`: constants of the clamped activation.  `names`: the checkpoint's names of gate, up and
        down behind the part's prefix (defaults: `gate_proj.weight`, ...)."""
        super().__init__()
        if activation not in _ACTIVATIONS and activation != _CLAMPED:
            raise ValueError(f"activation {activation!r} unknown (have {sorted(_ACTIVATIONS) + [_CLAMPED]})")
        if activation == _CLAMPED and (limit is None or limit <= 0):
            raise ValueError("the clamped activation needs a positive limit")
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.activation = activation
        self.limit = limit
        self.alpha = float(alpha)
        n = dict(gate="gate_proj.weight", up="up_proj.weight", down="down_proj.weight")
        n.update(names or {})
        self.names = n

    def param_decls(self):
        H, I, n = self.hidden_size, self.intermediate_size, self.names
        return {n["gate"]: ParamDecl((I, H)), n["up"]: ParamDecl((I, H)), n["down"]: ParamDecl((H, I))}

    def materialize(self, make):
        H, I, n = self.hidden_size, self.intermediate_size, self.names
        self.w_gate_up = make("gate_up_proj.weight", ParamDecl((2 * I, H)))
        self.tensors[n["gate"]] = self.w_gate_up[:I]
        self.tensors[n["up"]] = self.w_gate_up[I:]
        self.tensors[n["down"]] = make("down_proj.weight", ParamDecl((H, I)))

    def gated_weights(self):
        if self.activation == _CLAMPED:
            return None  # (the fused kernels know silu and gelu only)
        return self.w_gate_up, self.tensors[self.names["down"]], _ACTIVATIONS[self.activation]

    def activation_elems(self):
        return 3 * self.intermediate_size + self.hidden_size  # gate | up, their product, the output

    def forward(self, x, ctx):
        T = x.shape[0]
        I = self.intermediate_size
        gu = ctx.workspace.tokens("mlp.gate_up", T, 2 * I, x.dtype)
        act = ctx.workspace.tokens("mlp.act", T, I, x.dtype)
        if self.activation == _CLAMPED:
            linear(x, self.w_gate_up, gu)
            kernels().act_mul_clamped(gu, act, self.limit, self.alpha)
        else:
            kernels().linear_act_mul(x, self.w_gate_up, act, gu, _ACTIVATIONS[self.activation])
        out = ctx.workspace.tokens("ffn.out", T, self.hidden_size, x.dtype)
        linear(act, self.tensors[self.names["down"]], out)
        return out


@register_feed_forward("dense_mlp")
class DenseMLP(FeedForward):
    """down(act(up(x))) without a gate.  Activations: "xielu", with two learned numbers (p, q) in the tensor
    `act` [2]:

        z > 0:   softplus(p) z^2 + z / 2
        z <= 0:  (1/2 + softplus(q)) (e^z - 1 - z) + z / 2

    evaluated in 32-bit on the product's rounded output (csrc/sandwich_norm.cu)."""

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "xielu", names: dict | None = None):
        super().__init__()
        if activation != "xielu":
            raise ValueError(f"activation {activation!r} unknown (have ['xielu'])")
        if hidden_size <= 0 or intermediate_size <= 0:
            raise ValueError("sizes must be positive")
        self.hidden_size, self.intermediate_size, self.activation = hidden_size, intermediate_size, activation
        n = dict(up="up_proj.weight", down="down_proj.weight", act="act")
        n.update(names or {})
        self.names = n

    def param_decls(self):
        H, I, n = self.hidden_size, self.intermediate_size, self.names
        return {n["up"]: ParamDecl((I, H)), n["down"]: ParamDecl((H, I)), n["act"]: ParamDecl((2,), "bias32")}

    def activation_elems(self):
        return 2 * self.intermediate_size + self.hidden_size

    def forward(self, x, ctx):
        T, I, n = x.shape[0], self.intermediate_size, self.names
        u = ctx.workspace.tokens("mlp.up", T, I, x.dtype)
        linear(x, self.tensors[n["up"]], u)
        a = ctx.workspace.tokens("mlp.act", T, I, x.dtype)
        kernels().xielu(u, self.tensors[n["act"]], a)
        out = ctx.workspace.tokens("ffn.out", T, self.hidden_size, x.dtype)
        linear(a, self.tensors[n["down"]], out)
        return out
