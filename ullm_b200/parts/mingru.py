"""minGRU as a mixer with per-request state, and two mixers run side by side.

`mingru`: a gated recurrence per channel whose gates read only the current token.  With z = sigmoid(W_z h + b_z),
u = W_x h + b_x and the candidate c = u + 1/2 where u >= 0, sigmoid(u) where u < 0:

    S_t = (1 - z_t) S_{t-1} + z_t c_t           S_0 = 0
    out_t = W_o (S_t * silu(W_g h_t))

The three projections are ONE product with a 32-bit result; gates, candidate, state and the gated read-out are
32-bit in every engine dtype (csrc/mingru.cu).  The state, `width` floats, is one row per request slot in the
cache manager's state rows: zeroed when a slot is handed out, carried from step to step, so prompt portions of
any length and single decoded tokens continue one another.

`parallel_mixers`: result = left_scale * left(h) + right_scale * right(h) for two mixers that read the same rows.
Both stop in front of their output projections and leave their rows, already scaled, side by side in one buffer;
ONE product with the two projections' weights side by side [hidden, left width + right width] forms the sum.
At most one of the two keeps pages and at most one keeps state rows; each finds them in the execution's cache.
"""

from __future__ import annotations

import torch

from ..csrc import kernels
from .base import Mixer, ParamDecl, StateNeed
from .linear import linear
from .registry import build_mixer, register_mixer
from .window_attention import _ProjectsOutput


@register_mixer("mingru")
class MinGRU(Mixer, _ProjectsOutput):
    def __init__(self, hidden_size: int, width: int, names: dict | None = None):
        super().__init__()
        if hidden_size <= 0 or width <= 0:
            raise ValueError("sizes must be positive")
        self.hidden_size, self.width = hidden_size, width
        n = dict(z="z_proj.weight", z_bias="z_proj.bias", x="x_proj.weight", x_bias="x_proj.bias", g="g_proj.weight",
                 o="o_proj.weight")
        n.update(names or {})
        self.names = n

    def param_decls(self):
        H, W, n = self.hidden_size, self.width, self.names
        return {n["z"]: ParamDecl((W, H)), n["z_bias"]: ParamDecl((W,), "bias32"), n["x"]: ParamDecl((W, H)),
                n["x_bias"]: ParamDecl((W,), "bias32"), n["g"]: ParamDecl((W, H)), n["o"]: ParamDecl((H, W))}

    def materialize(self, make):
        H, W, n = self.hidden_size, self.width, self.names
        # one product for the gate's, the candidate's and the output gate's projections
        self.w_in = make("in_proj.weight", ParamDecl((3 * W, H)))
        self.tensors[n["z"]] = self.w_in[:W]
        self.tensors[n["x"]] = self.w_in[W:2 * W]
        self.tensors[n["g"]] = self.w_in[2 * W:]
        self.tensors[n["z_bias"]] = make(n["z_bias"], ParamDecl((W,), "bias32"))
        self.tensors[n["x_bias"]] = make(n["x_bias"], ParamDecl((W,), "bias32"))
        self.tensors[n["o"]] = self._make_o(make, n["o"], (H, W))

    def state_need(self):
        return StateNeed((self.width,), torch.float32)

    def activation_elems(self):
        # the 32-bit product (two elements' worth each in a 16-bit engine), the chunks' scratch, the read-out, the output
        return 6 * self.width + self.width + self.width + self.hidden_size

    def output_projection(self):
        return self.tensors[self.names["o"]], None

    def output_width(self) -> int:
        return self.width

    def forward(self, x, ctx, cache, project_output: bool = True, out=None, out_scale: float = 1.0):
        K = kernels()
        T, W, n, ws = x.shape[0], self.width, self.names, ctx.workspace
        if cache.state is None:
            raise RuntimeError("the minGRU mixer was given no state rows")
        azg = ws.tokens("mingru.in", T, 3 * W, torch.float32)
        K.linear_f32_out(x, self.w_in, azg)
        gated = out if out is not None else ws.tokens("mingru.gated", T, W, x.dtype)
        fold = None
        if ctx.max_q_len > K.mingru_chunk():
            # (a row per token is more than the chunks' pairs ever need: two floats per chunk and channel)
            fold = ws.tokens("mingru.fold", T, W, torch.float32)
        K.mingru(azg, 0, W, 2 * W, self.tensors[n["z_bias"]], self.tensors[n["x_bias"]], cache.state, ctx.cu_q,
                 ctx.req_slots, ctx.token_req, gated, out_scale, ctx.num_requests, ctx.max_q_len, fold)
        if not project_output:
            return gated
        res = ws.tokens("mixer.out", T, self.hidden_size, x.dtype)
        linear(gated, self.tensors[n["o"]], res)
        return res


@register_mixer("parallel_mixers")
class ParallelMixers(Mixer):
    def __init__(self, hidden_size: int, left, right, left_scale: float = 1.0, right_scale: float = 1.0,
                 names: dict | None = None):
        """`left`, `right`: `MixerSpec`s of mixers that can stop in front of their output projection
        (`forward(..., project_output=False, out=, out_scale=)`, `output_width()`, a shareable `o` weight).
        `names`: the prefixes of the two mixers' tensors behind this mixer's own prefix."""
        super().__init__()
        self.hidden_size = hidden_size
        self.left, self.right = build_mixer(left), build_mixer(right)
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        for m in (self.left, self.right):
            if not isinstance(m, _ProjectsOutput):
                raise ValueError(f"{type(m).__name__} cannot hand its output projection to a caller")
        if sum(m.cache_need() is not None for m in (self.left, self.right)) > 1:
            raise ValueError("at most one of two mixers side by side keeps pages")
        if sum(m.state_need() is not None for m in (self.left, self.right)) > 1:
            raise ValueError("at most one of two mixers side by side keeps state rows")
        n = dict(left="left.", right="right.")
        n.update(names or {})
        self.names = n

    def subparts(self):
        return {self.names["left"]: self.left, self.names["right"]: self.right}

    def materialize(self, make):
        # (runs before the two mixers' own `materialize`: they then find their share of the wide matrix)
        wl, wr = self.left.output_width(), self.right.output_width()
        self.w_o = make("o_proj.weight", ParamDecl((self.hidden_size, wl + wr)))
        self.left.shared_o = self.w_o[:, :wl]
        self.right.shared_o = self.w_o[:, wl:]

    def cache_need(self):
        return self.left.cache_need() or self.right.cache_need()

    def aux_cache_need(self):
        return self.left.aux_cache_need() or self.right.aux_cache_need()

    def state_need(self):
        return self.left.state_need() or self.right.state_need()

    def graph_key(self, ctx):
        return (self.left.graph_key(ctx), self.right.graph_key(ctx))

    def graph_key_group(self):
        return (type(self), self.left.graph_key_group(), self.right.graph_key_group())

    def activation_elems(self):
        return (self.left.activation_elems() + self.right.activation_elems() + self.left.output_width()
                + self.right.output_width() + self.hidden_size)

    def output_projection(self):
        return self.w_o, None

    def forward(self, x, ctx, cache):
        T = x.shape[0]
        wl, wr = self.left.output_width(), self.right.output_width()
        both = ctx.workspace.tokens("parallel.rows", T, wl + wr, x.dtype)
        self.left.forward(x, ctx, cache, project_output=False, out=both[:, :wl], out_scale=self.left_scale)
        self.right.forward(x, ctx, cache, project_output=False, out=both[:, wl:], out_scale=self.right_scale)
        out = ctx.workspace.tokens("mixer.out", T, self.hidden_size, x.dtype)
        linear(both, self.w_o, out)
        return out
