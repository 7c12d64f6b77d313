"""Routed feed-forward: a router picks `top` of `num_experts` small gated feed-forwards per token.

    z = W_router h (32-bit);  s = sigmoid(z) (or softmax over the experts);  the `top` largest s are chosen;
    weight c = s of the chosen (optionally renormalized to sum 1);
    y = sum over the chosen of  expert(c h)   (`weight_on` = "input")   or   c expert(h)   ("output"),
    expert(x) = W_down (act(W_gate x) * (W_up x)),  no biases.

Options: `correction` (a vector `correction` over the router's outputs that is added to the scores for the CHOICE
only; the weights stay the scores); `identity` n (the router has n more outputs behind the experts', standing for
experts without tensors whose output is their input: a token that picks one gets weight x its own row); the clamped
activation g' sigmoid(alpha g') (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit); `shared` (a feed-forward
of its own, run for every token and added, with `shared_gate` times sigmoid(w_sg . h), one number per token, whose
row rides behind the router's in one 32-bit product).

The experts' matrices live stacked ([experts, 2 I, hidden] with gate rows on up rows, and [experts, hidden, I]);
the checkpoint's per-expert tensors are views of the stacks.  Nothing of the routing comes back to the host: the
(token, choice) pairs are grouped by expert on the device and a grouped product runs over the groups, so a decode
step with this feed-forward can be recorded into a CUDA graph.
"""

from __future__ import annotations

import torch

from ..csrc import kernels
from .base import FeedForward, ParamDecl
from .registry import build_feed_forward, register_feed_forward

_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "swiglu_clamped": 2}


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, top: int, activation: str = "silu",
                 scores: str = "sigmoid", renormalize: bool = False, weight_on: str = "output",
                 names: dict | None = None, limit: float | None = None, alpha: float = 1.702, correction: bool = False,
                 identity: int = 0, shared=None, shared_gate: bool = False):
        """`names`: router, correction, shared (a prefix), shared_gate, and per expert (format strings taking the
        expert's number) gate, up, down.  `shared`: a `FeedForwardSpec`."""
        super().__init__()
        if activation not in _ACTIVATIONS:
            raise ValueError(f"activation {activation!r} unknown (have {sorted(_ACTIVATIONS)})")
        if activation == "swiglu_clamped" and (limit is None or not limit > 0):
            raise ValueError("the clamped activation needs a positive limit")
        if identity < 0 or (identity and weight_on != "output"):
            raise ValueError("experts that pass their input: a count, with the weight on the output")
        if shared_gate and shared is None:
            raise ValueError("a gate of the shared expert without a shared expert")
        if scores not in ("sigmoid", "softmax") or weight_on not in ("input", "output"):
            raise ValueError("scores: 'sigmoid' or 'softmax'; weight_on: 'input' or 'output'")
        if not 0 < top <= num_experts + identity or top > 32 or num_experts + identity > 1024:
            raise ValueError(f"top={top} of {num_experts} + {identity} experts: the kernels take top <= 32 and up to "
                             f"1024 router outputs")
        self.H, self.I, self.E, self.top = hidden_size, intermediate_size, num_experts, top
        self.activation, self.scores, self.renormalize, self.weight_on = activation, scores, bool(renormalize), weight_on
        self.limit, self.alpha = float(limit or 0.0), float(alpha)
        self.correction, self.identity = bool(correction), int(identity)
        self.R = num_experts + self.identity  # the router's outputs
        self.shared = build_feed_forward(shared) if shared is not None else None
        self.shared_gate = bool(shared_gate)
        n = dict(router="router.weight", gate="experts.{}.gate_proj.weight", up="experts.{}.up_proj.weight",
                 down="experts.{}.down_proj.weight", correction="router.correction", shared="shared.",
                 shared_gate="shared_gate.weight")
        n.update(names or {})
        self.names = n

    def subparts(self):
        return {self.names["shared"]: self.shared} if self.shared is not None else {}

    def param_decls(self):
        n = self.names
        d = {n["router"]: ParamDecl((self.R, self.H))}
        if self.correction:
            d[n["correction"]] = ParamDecl((self.R,), "bias32")
        if self.shared_gate:
            d[n["shared_gate"]] = ParamDecl((1, self.H))
        for e in range(self.E):
            d[n["gate"].format(e)] = ParamDecl((self.I, self.H))
            d[n["up"].format(e)] = ParamDecl((self.I, self.H))
            d[n["down"].format(e)] = ParamDecl((self.H, self.I))
        return d

    def materialize(self, make):
        n, E, I, H = self.names, self.E, self.I, self.H
        # the router's rows, and behind them the row of the shared expert's gate: one product with a 32-bit result.
        # Rows of zeros fill the matrix up to a multiple of 8, so that the result's rows start on 16-byte borders
        # (the library has no fast product for other strides)
        used = self.R + (1 if self.shared_gate else 0)
        self.w_router = make(n["router"], ParamDecl((-(-used // 8) * 8, H)))
        self.w_router[used:].zero_()
        self.tensors[n["router"]] = self.w_router[:self.R]
        if self.shared_gate:
            self.tensors[n["shared_gate"]] = self.w_router[self.R:used]
        self.w_correction = None
        if self.correction:
            self.w_correction = self.tensors[n["correction"]] = make(n["correction"], ParamDecl((self.R,), "bias32"))
        self.w_gate_up = make("experts.gate_up.weight", ParamDecl((E, 2 * I, H)))
        self.w_down = make("experts.down.weight", ParamDecl((E, H, I)))
        for e in range(E):
            self.tensors[n["gate"].format(e)] = self.w_gate_up[e, :I]
            self.tensors[n["up"].format(e)] = self.w_gate_up[e, I:]
            self.tensors[n["down"].format(e)] = self.w_down[e]

    def activation_elems(self):
        shared = self.shared.activation_elems() if self.shared is not None else 0
        return self.top * (self.I + self.H) + self.H + self.R + 1 + shared

    def forward(self, x, ctx):
        return self._run(x, ctx, None)

    def forward_add(self, x, ctx, stream, scale=None, next_norm=None) -> bool:
        """stream (32-bit, in place) += scale * forward(x), the experts' weighted sum never leaving 32-bit, and
        `next_norm` = (weight, eps, out): the RMS norm of the updated stream's rows in `out` (which may be x itself).
        False when this part cannot (nothing has run then): the caller then adds `forward(x)` itself."""
        if self.weight_on != "output" or stream.shape[1] * 4 > 160 * 1024:
            return False
        self._run(x, ctx, (stream, scale, next_norm))
        return True

    def _run(self, x, ctx, add):
        K = kernels()
        T, top, E = x.shape[0], self.top, self.E
        ws = ctx.workspace
        logits = ws.tokens("moe.logits", T, self.w_router.shape[0], torch.float32)
        K.linear_f32_out(x, self.w_router, logits)
        choice = ws.tokens("moe.choice", T, top, torch.int32)
        weight = ws.tokens("moe.weight", T, top, torch.float32)
        K.moe_route(logits, choice, weight, top, self.scores == "softmax", self.renormalize,
                    correction=self.w_correction, experts=self.R)
        offsets = ws.get("moe.offsets", 1, E + 1, torch.int32)
        order = ws.tokens("moe.sorted", T, top, torch.int32)
        place = ws.tokens("moe.place", T, top, torch.int32)
        K.moe_arrange(choice, T * top, E, offsets, order, place)
        act = ws.tokens("moe.act", T * top, self.I, x.dtype) if top == 1 else ws.get("moe.act", T * top, self.I, x.dtype, reserve=ws.max_tokens * top)
        rows = ws.tokens("moe.rows", T * top, self.H, x.dtype) if top == 1 else ws.get("moe.rows", T * top, self.H, x.dtype, reserve=ws.max_tokens * top)
        on_input = self.weight_on == "input"
        # (a choice at or beyond E, an expert that passes its input, gets no place: `moe_arrange` skips it)
        K.moe_grouped_linear(x, self.w_gate_up, offsets, order, weight if on_input else None, act, top, True, True,
                             _ACTIVATIONS[self.activation], self.limit, self.alpha)
        K.moe_grouped_linear(act, self.w_down, offsets, order, None, rows, top, False, False)
        shared = None
        if self.shared is not None:
            shared = (self.shared.forward(x, ctx), logits[:, self.R:self.R + 1] if self.shared_gate else None)
        passing = (choice, E, x) if self.identity else None
        if add is not None:
            stream, scale, next_norm = add
            if not K.moe_combine_add_norm(rows, place, None if on_input else weight, top, stream, scale, next_norm,
                                          passing=passing, shared=shared):
                raise RuntimeError("the combining kernel refused a row length that had been accepted")
            return None
        # (a buffer of its own: the shared expert's output may lie in "ffn.out")
        out = ws.tokens("moe.out", T, self.H, x.dtype)
        K.moe_combine(rows, place, None if on_input else weight, out, top, passing=passing, shared=shared)
        return out
