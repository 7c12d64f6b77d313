"""Arrangement of a layer: pre-norm, residual stream.

ullm/models/qwen3.py:160-178: the stream is carried as (x, residual).  The
first block takes residual = x; afterwards each norm is the fused form
"residual <- x + residual (32-bit sum, rounded on store); h = norm(sum)".
"""

from __future__ import annotations

import torch

from ..csrc import kernels
from .base import Block, Norm, ParamDecl
from .linear import linear
from .registry import build_norm, register_block


@register_block("prenorm_residual")
class PreNormResidualBlock(Block):
    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm, names=None):
        super().__init__()
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm
        n = names or {}
        self.names = {
            "mixer": n.get("mixer", "mixer."),
            "feed_forward": n.get("feed_forward", "feed_forward."),
            "mixer_norm": n.get("mixer_norm", "mixer_norm."),
            "feed_forward_norm": n.get("feed_forward_norm", "feed_forward_norm."),
        }

    def subparts(self):
        return {
            self.names["mixer_norm"]: self.mixer_norm,
            self.names["mixer"]: self.mixer,
            self.names["feed_forward_norm"]: self.feed_forward_norm,
            self.names["feed_forward"]: self.feed_forward,
        }

    def activation_elems(self):
        # the normed rows, and the wider of the two sub-layers (they run one after the other)
        size = getattr(self.mixer_norm, "size", 0)
        return size + max(self.mixer.activation_elems(), self.feed_forward.activation_elems())

    takes_next_norm = True  # `forward` accepts the norm that the next block (or nobody) will apply first

    def accepts_folded_norm(self) -> bool:
        """True when this block can start from an operand r * w and the rows' sums of squares that the block
        before left (instead of norming r itself): an RMSNorm in front of a mixer whose first step is a product."""
        return self.mixer_norm.rms_params() is not None and self.mixer.takes_input_norm()

    def forward(self, x, residual, ctx, cache, next_norm=None):
        """x: the previous sub-layer's output that is still to be added to the stream (the embedding for the
        first block, with residual None; None when nothing is pending).  Returns (feed-forward output or None,
        residual); the caller's next norm adds them.  `next_norm`: the norm the next block will apply to the
        stream first, if that block `accepts_folded_norm()`; in small decode steps this block's last product then
        prepares it (`ctx.folded_norm`), and the next block's mixer starts from that."""
        pending = x if x is not None else residual
        T = pending.shape[0]
        folded, ctx.folded_norm = getattr(ctx, "folded_norm", None), None
        input_norm = None
        fused = chain = None
        if ctx.decode_only and residual is not None:
            fused = self._fusable_tail(T, residual)
            chain = self._fusable_chain(T, residual) if fused is None else None
        if (folded is not None and folded[0] is self.mixer_norm and x is None and residual is not None
                and chain is not None):
            # the block before left r * w and the sums of squares: the mixer's first product applies 1 / rms
            _norm, h, sq, eps = folded
            input_norm = (sq, residual.shape[1], eps)
        else:
            h = ctx.workspace.tokens("block.normed", T, pending.shape[1], pending.dtype)
            if residual is None:
                residual = x
                self.mixer_norm.forward(x, None, out=h)
            elif x is None:
                self.mixer_norm.forward(residual, None, out=h)
            else:
                self.mixer_norm.forward(x, residual, out=h)
        if fused is None and chain is None and ctx.decode_only:
            fused = self._fusable_tail(T, residual)  # the first block: the stream has only now got its rows
            chain = self._fusable_chain(T, residual) if fused is None else None
        if fused is not None:
            # few rows (decode steps): output projection, residual, norm, gated feed-forward and residual in one
            # kernel; the stream then holds everything and nothing is pending
            w_o, norm_w, eps, w_gate_up, w_down, act = fused
            a = self.mixer.forward(h, ctx, cache, project_output=False)
            work = ctx.workspace.tokens("mlp.act", T, w_down.shape[1], residual.dtype)
            kernels().fused_layer_tail(a, residual, work, w_o, w_gate_up, w_down, norm_w, eps, act)
            return None, residual
        if chain is not None:
            # few rows, every product the weight-streaming kernel: the output projection adds the residual itself
            # and leaves r * w and the sums of squares for the norm, the gate / up product applies 1 / rms to its
            # sums, the down projection adds the residual (and prepares the next block's norm the same way):
            # three kernels, no norm kernel, nothing pending
            K, (w_o, norm_w, eps, w_gate_up, w_down, act) = kernels(), chain
            if input_norm is not None:
                a = self.mixer.forward(h, ctx, cache, project_output=False, input_norm=input_norm)
            else:
                a = self.mixer.forward(h, ctx, cache, project_output=False)
            H = residual.shape[1]
            hn = ctx.workspace.tokens("block.normed", T, H, residual.dtype)
            sq = ctx.workspace.get("block.norm_sq", 1, K.stream_sq_floats(H), torch.float32)
            work = ctx.workspace.tokens("mlp.act", T, w_down.shape[1], residual.dtype)
            behind = None
            nxt = next_norm.rms_params() if next_norm is not None else None
            if nxt is not None and nxt[0].numel() == H and K.chain_norms >= 2:
                operand = ctx.workspace.tokens("block.next_operand", T, H, residual.dtype)
                sq2 = ctx.workspace.get("block.next_sq", 1, K.stream_sq_floats(H), torch.float32)
                behind = (nxt[0], operand, sq2)
            if (K.stream_linear(a, w_o, residual, None, None, residual, norm_behind=(norm_w, hn, sq))
                    and K.stream_linear(hn, w_gate_up, work, None, act, norm_in_front=(sq, H, eps))
                    and K.stream_linear(work, w_down, residual, None, None, residual, norm_behind=behind)):
                if behind is not None:
                    ctx.folded_norm = (next_norm, behind[1], behind[2], nxt[1])
                return None, residual
            raise RuntimeError("the chained products were refused after the sizes had been accepted")
        a = self.mixer.forward(h, ctx, cache)
        self.feed_forward_norm.forward(a, residual, out=h)
        y = self.feed_forward.forward(h, ctx)
        return y, residual

    def _fusable_chain(self, rows: int, residual):
        """The same parts as `_fusable_tail` needs, when the step's products are all the stream kernel."""
        if not residual.is_cuda or not kernels().stream_chain_applies(rows, residual.dtype):
            return None
        proj, norm, ffn = self.mixer.output_projection(), self.feed_forward_norm.rms_params(), self.feed_forward.gated_weights()
        if proj is None or norm is None or ffn is None or proj[1] is not None:
            return None
        w_o, (norm_w, eps), (w_gate_up, w_down, act) = proj[0], norm, ffn
        K = kernels()
        H = residual.shape[1]
        if (w_o.dtype != torch.bfloat16 or H % 8 or w_o.shape[1] % 8 or w_down.shape[1] % 8
                or not K.lib.ullm_linear_stream_supported(rows, H, w_o.shape[1])):
            return None
        return w_o, norm_w, eps, w_gate_up, w_down, act

    def _fusable_tail(self, rows: int, residual):
        """What the fused kernel needs, if this block's parts offer it (a mixer that ends in a bias-free linear
        map, an RMSNorm, a bias-free gated feed-forward) and the kernel takes the sizes; else None."""
        proj, norm, ffn = self.mixer.output_projection(), self.feed_forward_norm.rms_params(), self.feed_forward.gated_weights()
        if proj is None or norm is None or ffn is None or proj[1] is not None or not residual.is_cuda:
            return None
        w_o, (norm_w, eps), (w_gate_up, w_down, act) = proj[0], norm, ffn
        if not kernels().layer_tail_applies(rows, residual.dtype, residual.shape[1], w_o.shape[1], w_down.shape[1]):
            return None
        return w_o, norm_w, eps, w_gate_up, w_down, act


@register_block("outnorm_residual")
class OutputNormResidualBlock(Block):
    """The norm sits on each sub-layer's OUTPUT, and the normed output is added to the stream with a multiplier:

        x <- x + mult * norm_a(mixer(x));   x <- x + mult * norm_b(feed_forward(x))

    Both sub-layers read the stream itself.  The stream is 32-bit whatever the engine's dtype (the model is built
    with `stream_dtype="float32"`); the sub-layers' operand is the stream rounded to the engine's dtype, which the
    kernel that updates the stream writes beside it (`ctx.stream_operand`).  A layer may have no feed-forward."""

    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm, names=None, residual_mult: float = 1.0):
        super().__init__()
        if (feed_forward is None) != (feed_forward_norm is None):
            raise ValueError("a feed-forward and its norm come together or not at all")
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm
        self.residual_mult = float(residual_mult)
        n = names or {}
        self.names = {
            "mixer": n.get("mixer", "mixer."),
            "feed_forward": n.get("feed_forward", "feed_forward."),
            "mixer_norm": n.get("mixer_norm", "mixer_norm."),
            "feed_forward_norm": n.get("feed_forward_norm", "feed_forward_norm."),
        }

    def subparts(self):
        s = {self.names["mixer_norm"]: self.mixer_norm, self.names["mixer"]: self.mixer}
        if self.feed_forward is not None:
            s[self.names["feed_forward_norm"]] = self.feed_forward_norm
            s[self.names["feed_forward"]] = self.feed_forward
        return s

    def activation_elems(self):
        ff = self.feed_forward.activation_elems() if self.feed_forward is not None else 0
        return 3 * getattr(self.mixer_norm, "size", 0) + max(self.mixer.activation_elems(), ff)

    def forward(self, x, residual, ctx, cache):
        """The stream arrives as `x` (first block, residual None) or as `residual` (x None); returns (None, stream)."""
        stream = residual if residual is not None else x
        if stream.dtype != torch.float32:
            raise RuntimeError("this block takes a 32-bit residual stream (ModelSpec.stream_dtype='float32')")
        T, H = stream.shape
        h = ctx.stream_operand
        if h is None or h.shape != stream.shape:
            engine_dtype = self.mixer.operand_dtype()
            if engine_dtype == torch.float32:
                h = stream
            else:
                h = ctx.workspace.tokens("model.stream_copy", T, H, engine_dtype)
                kernels().cast_rows_f32(stream, h)
        copy = None if h is stream else h
        a = self.mixer.forward(h, ctx, cache)
        self.mixer_norm.scale_add(a, stream, self.residual_mult, copy)
        if self.feed_forward is not None:
            y = self.feed_forward.forward(h, ctx)
            self.feed_forward_norm.scale_add(y, stream, self.residual_mult, copy)
        ctx.stream_operand = h
        return None, stream


@register_block("parallel_gated")
class ParallelGatedBlock(Block):
    """Mixer and feed-forward read the same normed stream and are added to it together:

        h = norm(x);   x <- x + (g1 * mixer(h) + g2 * feed_forward(h))

    with g_i = sigmoid(R_i h + b_i) element by element when `gated` (else 1), and, when `side_dim` > 0, a
    per-layer token input behind it: with e the layer's share (`side_index`) of the model's token side table,

        y = P (gelu_tanh(G x) * e);   x <- x + n * y / sqrt(mean(y^2) + eps)

    The stream is 32-bit whatever the engine's dtype (the model is built with `stream_dtype="float32"`); the gates'
    projections are ONE product with a 32-bit result, and sigmoids, sums and norms are 32-bit.  A layer may have no
    feed-forward (then no second gate either).  `feed_forward_norm` is unused: there is one norm."""

    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm, names=None, gated: bool = True,
                 side_dim: int = 0, side_index: int = 0, eps: float = 1e-6):
        super().__init__()
        if feed_forward_norm is not None:
            raise ValueError("a parallel block has one norm (feed_forward_norm must be None)")
        if not gated:
            raise ValueError("the parallel block without gates is not built (gated=True)")
        self.mixer, self.feed_forward, self.mixer_norm = mixer, feed_forward, mixer_norm
        self.gated, self.side_dim, self.side_index, self.eps = bool(gated), int(side_dim), int(side_index), float(eps)
        self.hidden_size = mixer_norm.size
        n = dict(mixer="mixer.", feed_forward="feed_forward.", mixer_norm="norm.", gate1="gate1.weight",
                 gate1_bias="gate1.bias", gate2="gate2.weight", gate2_bias="gate2.bias", side_gate="side.gate",
                 side_proj="side.proj", side_norm="side.norm")
        n.update(names or {})
        self.names = n

    def subparts(self):
        s = {self.names["mixer_norm"]: self.mixer_norm, self.names["mixer"]: self.mixer}
        if self.feed_forward is not None:
            s[self.names["feed_forward"]] = self.feed_forward
        return s

    def param_decls(self):
        W, n, d = self.hidden_size, self.names, {}
        if self.gated:
            d[n["gate1"]] = ParamDecl((W, W))
            d[n["gate1_bias"]] = ParamDecl((W,), "bias32")
            if self.feed_forward is not None:
                d[n["gate2"]] = ParamDecl((W, W))
                d[n["gate2_bias"]] = ParamDecl((W,), "bias32")
        if self.side_dim:
            d[n["side_gate"]] = ParamDecl((self.side_dim, W))
            d[n["side_proj"]] = ParamDecl((W, self.side_dim))
            d[n["side_norm"]] = ParamDecl((W,), "norm")
        return d

    def materialize(self, make):
        W, n = self.hidden_size, self.names
        self.w_gates = None
        if self.gated:
            two = self.feed_forward is not None
            # the two gates' projections as one matrix with rows gate1 | gate2
            self.w_gates = make("gates.weight", ParamDecl(((2 if two else 1) * W, W)))
            self.tensors[n["gate1"]] = self.w_gates[:W]
            self.tensors[n["gate1_bias"]] = make(n["gate1_bias"], ParamDecl((W,), "bias32"))
            if two:
                self.tensors[n["gate2"]] = self.w_gates[W:]
                self.tensors[n["gate2_bias"]] = make(n["gate2_bias"], ParamDecl((W,), "bias32"))
        if self.side_dim:
            self.tensors[n["side_gate"]] = make(n["side_gate"], ParamDecl((self.side_dim, W)))
            self.tensors[n["side_proj"]] = make(n["side_proj"], ParamDecl((W, self.side_dim)))
            self.tensors[n["side_norm"]] = make(n["side_norm"], ParamDecl((W,), "norm"))

    def activation_elems(self):
        W = self.hidden_size
        ff = self.feed_forward.activation_elems() if self.feed_forward is not None else 0
        # the normed rows, the stream's copy, both sub-layers at once, the gates in 32-bit, the side input
        return 2 * W + self.mixer.activation_elems() + ff + 4 * W + 2 * self.side_dim + W

    takes_next_norm = True  # `forward` accepts the norm that the next block will apply first

    def accepts_folded_norm(self) -> bool:
        """True: this block can start from normed rows that the block before left in `ctx.prepared_norm`."""
        return self.mixer_norm.rms_params() is not None

    def forward(self, x, residual, ctx, cache, next_norm=None):
        """The stream arrives as `x` (first block, residual None) or as `residual` (x None); returns (None, stream).
        `next_norm`: the norm the next block applies first; with a token side input the kernel that adds it to the
        stream also leaves that norm's rows (`ctx.prepared_norm`), which a block of this kind then starts from."""
        K = kernels()
        stream = residual if residual is not None else x
        if stream.dtype != torch.float32:
            raise RuntimeError("this block takes a 32-bit residual stream (ModelSpec.stream_dtype='float32')")
        T, W = stream.shape
        n, ws = self.names, ctx.workspace
        dt = self.mixer.operand_dtype()
        prepared, ctx.prepared_norm = getattr(ctx, "prepared_norm", None), None
        if prepared is not None and prepared[0] is self.mixer_norm and prepared[1].shape == (T, W):
            h = prepared[1]
        else:
            h = ws.tokens("block.normed", T, W, dt)
            self.mixer_norm.forward_rows(stream, None, h)
        a = self.mixer.forward(h, ctx, cache)
        f = self.feed_forward.forward(h, ctx) if self.feed_forward is not None else None
        copy = ws.tokens("model.stream_copy", T, W, dt) if (self.side_dim and dt != torch.float32) else None
        gates = ws.tokens("block.gates", T, self.w_gates.shape[0], torch.float32)
        K.linear_f32_out(h, self.w_gates, gates)
        K.gated_add_f32(a, f, gates, self.tensors[n["gate1_bias"]],
                        self.tensors[n["gate2_bias"]] if f is not None else None, stream, copy)
        if self.side_dim:
            side = ctx.token_side
            if side is None or side.dim != self.side_dim or not 0 <= self.side_index < side.shares:
                raise RuntimeError("this block's per-layer token input does not fit the model's token side table")
            operand = copy if copy is not None else stream
            s = ws.tokens("block.side_gate", T, self.side_dim, dt)
            linear(operand, self.tensors[n["side_gate"]], s)
            g = ws.tokens("block.side_in", T, self.side_dim, dt)
            last = ctx.last_tokens
            K.side_gate_mul(s, ctx.token_ids, side.table, self.side_index * self.side_dim, g, last,
                            ctx.token_req if last is not None else None, ctx.req_slots if last is not None else None)
            y = ws.tokens("block.side_out", T, W, dt)
            linear(g, self.tensors[n["side_proj"]], y)
            nxt = next_norm.rms_params() if next_norm is not None else None
            done = False
            if nxt is not None and nxt[0].numel() == W:
                # (all of this block's readers of h are done: the next block's rows take its place)
                h_next = ws.tokens("block.normed", T, W, dt)
                done = K.norm_scale_add(y, stream, self.tensors[n["side_norm"]], self.eps, 1.0, None,
                                        next_norm=(nxt[0], nxt[1], h_next))
                if done:
                    ctx.prepared_norm = (next_norm, h_next)
            if not done:
                K.norm_scale_add(y, stream, self.tensors[n["side_norm"]], self.eps, 1.0, None)
        ctx.stream_operand = None
        return None, stream


@register_block("sandwich_residual")
class SandwichResidualBlock(Block):
    """A norm on BOTH sides of each sub-layer, on a 32-bit residual stream:

        x <- x + norm_1b(mixer(norm_1(x)));   x <- x + norm_2b(feed_forward(norm_2(x)))

    `mixer_norm` / `feed_forward_norm` are the norms in front, `mixer_out_norm` / `feed_forward_out_norm`
    (`NormSpec`s among the block's arguments) the ones behind.  A layer may have no feed-forward (and then neither
    of its norms).  The norms must offer `row_params()`: one kernel norms a sub-layer's output, adds it to the
    stream and leaves the rows of the norm that reads the stream next (this block's second one, or the next
    block's first, `ctx.prepared_norm`), so the stream is read and written once per sub-layer."""

    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm, names=None, mixer_out_norm=None,
                 feed_forward_out_norm=None):
        super().__init__()
        if mixer_out_norm is None:
            raise ValueError("this arrangement norms the mixer's output too (mixer_out_norm)")
        if not ((feed_forward is None) == (feed_forward_norm is None) == (feed_forward_out_norm is None)):
            raise ValueError("a feed-forward and its two norms come together or not at all")
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self.mixer_out_norm = build_norm(mixer_out_norm)
        self.feed_forward_out_norm = build_norm(feed_forward_out_norm) if feed_forward_out_norm is not None else None
        for nm in (self.mixer_norm, self.mixer_out_norm, self.feed_forward_norm, self.feed_forward_out_norm):
            if nm is not None and not hasattr(nm, "row_params"):
                raise ValueError(f"{type(nm).__name__} cannot be folded into the stream's row kernels")
        self.hidden_size = mixer_norm.size
        n = dict(mixer="mixer.", feed_forward="feed_forward.", mixer_norm="mixer_norm.",
                 mixer_out_norm="mixer_out_norm.", feed_forward_norm="feed_forward_norm.",
                 feed_forward_out_norm="feed_forward_out_norm.")
        n.update(names or {})
        self.names = n

    def subparts(self):
        n = self.names
        s = {n["mixer_norm"]: self.mixer_norm, n["mixer_out_norm"]: self.mixer_out_norm, n["mixer"]: self.mixer}
        if self.feed_forward is not None:
            s[n["feed_forward_norm"]] = self.feed_forward_norm
            s[n["feed_forward_out_norm"]] = self.feed_forward_out_norm
            s[n["feed_forward"]] = self.feed_forward
        return s

    def activation_elems(self):
        ff = self.feed_forward.activation_elems() if self.feed_forward is not None else 0
        return 3 * self.hidden_size + max(self.mixer.activation_elems(), ff)

    takes_next_norm = True  # `forward` accepts the norm that the next block will apply first

    def accepts_folded_norm(self) -> bool:
        """True: this block can start from normed rows that whoever updated the stream last left in
        `ctx.prepared_norm`."""
        return self.mixer_norm.row_params() is not None

    def forward(self, x, residual, ctx, cache, next_norm=None):
        """The stream arrives as `x` (first block, residual None) or as `residual` (x None); returns (None, stream)."""
        K = kernels()
        stream = residual if residual is not None else x
        if stream.dtype != torch.float32:
            raise RuntimeError("this block takes a 32-bit residual stream (ModelSpec.stream_dtype='float32')")
        T, W = stream.shape
        ws = ctx.workspace
        dt = self.mixer.operand_dtype()
        prepared, ctx.prepared_norm = getattr(ctx, "prepared_norm", None), None
        if prepared is not None and prepared[0] is self.mixer_norm and prepared[1].shape == (T, W):
            h = prepared[1]
        else:
            h = ws.tokens("block.normed", T, W, dt)
            self.mixer_norm.forward_rows(stream, None, h)
        a = self.mixer.forward(h, ctx, cache)
        nxt = next_norm.row_params() if (next_norm is not None and hasattr(next_norm, "row_params")) else None
        if nxt is not None and nxt[0].numel() != W:
            nxt = None
        # (every reader of h is done when the kernel that overwrites it runs: the rows take its place)
        h2 = ws.tokens("block.normed", T, W, dt)
        w, eps, center = self.mixer_out_norm.row_params()
        if self.feed_forward is not None:
            K.norm_add_norm(stream, a, w, eps, 1.0, center, next_norm=(*self.feed_forward_norm.row_params(), h2))
            f = self.feed_forward.forward(h2, ctx)
            w, eps, center = self.feed_forward_out_norm.row_params()
            K.norm_add_norm(stream, f, w, eps, 1.0, center, next_norm=(*nxt, h2) if nxt is not None else None)
        else:
            K.norm_add_norm(stream, a, w, eps, 1.0, center, next_norm=(*nxt, h2) if nxt is not None else None)
        if nxt is not None:
            ctx.prepared_norm = (next_norm, h2)
        ctx.stream_operand = None
        return None, stream


@register_block("prenorm_scaled")
class PreNormScaledBlock(Block):
    """A pre-norm layer on a 32-bit residual stream, with an optional scale per channel on each sub-layer's output:

        x <- x + s1 * mixer(norm_1(x));   x <- x + s2 * feed_forward(norm_2(x))

    (`layer_scale` False: s1 = s2 = 1 and no tensors for them.)  A layer may have no feed-forward (then neither its
    norm nor its scale).  The norms must offer `row_params()`: the kernel that adds a sub-layer's scaled output to the
    stream also leaves the rows of the norm that reads the stream next (this block's second one, or the next block's
    first, `ctx.prepared_norm`), so the stream is read and written once per sub-layer.  The sum is 32-bit; the
    sub-layers' operands are the normed rows rounded to the engine's dtype."""

    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm, names=None, layer_scale: bool = False):
        super().__init__()
        if (feed_forward is None) != (feed_forward_norm is None):
            raise ValueError("a feed-forward and its norm come together or not at all")
        for nm in (mixer_norm, feed_forward_norm):
            if nm is not None and (not hasattr(nm, "row_params") or nm.row_params.__func__ is Norm.row_params):
                raise ValueError(f"{type(nm).__name__} cannot be folded into the stream's row kernels")
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self.layer_scale = bool(layer_scale)
        self.hidden_size = mixer_norm.size
        n = dict(mixer="mixer.", feed_forward="feed_forward.", mixer_norm="mixer_norm.",
                 feed_forward_norm="feed_forward_norm.", mixer_scale="mixer_scale", feed_forward_scale="feed_forward_scale")
        n.update(names or {})
        self.names = n

    def subparts(self):
        n = self.names
        s = {n["mixer_norm"]: self.mixer_norm, n["mixer"]: self.mixer}
        if self.feed_forward is not None:
            s[n["feed_forward_norm"]] = self.feed_forward_norm
            s[n["feed_forward"]] = self.feed_forward
        return s

    def param_decls(self):
        if not self.layer_scale:
            return {}
        d = {self.names["mixer_scale"]: ParamDecl((self.hidden_size,), "norm")}
        if self.feed_forward is not None:
            d[self.names["feed_forward_scale"]] = ParamDecl((self.hidden_size,), "norm")
        return d

    def activation_elems(self):
        ff = self.feed_forward.activation_elems() if self.feed_forward is not None else 0
        return 3 * self.hidden_size + max(self.mixer.activation_elems(), ff)

    takes_next_norm = True  # `forward` accepts the norm that the next block will apply first

    def accepts_folded_norm(self) -> bool:
        """True: this block can start from normed rows that whoever updated the stream last left in
        `ctx.prepared_norm`."""
        return self.mixer_norm.row_params() is not None

    def forward(self, x, residual, ctx, cache, next_norm=None):
        """The stream arrives as `x` (first block, residual None) or as `residual` (x None); returns (None, stream)."""
        K = kernels()
        stream = residual if residual is not None else x
        if stream.dtype != torch.float32:
            raise RuntimeError("this block takes a 32-bit residual stream (ModelSpec.stream_dtype='float32')")
        T, W = stream.shape
        ws = ctx.workspace
        dt = self.mixer.operand_dtype()
        prepared, ctx.prepared_norm = getattr(ctx, "prepared_norm", None), None
        if prepared is not None and prepared[0] is self.mixer_norm and prepared[1].shape == (T, W):
            h = prepared[1]
        else:
            h = ws.tokens("block.normed", T, W, dt)
            self.mixer_norm.forward_rows(stream, None, h)
        a = self.mixer.forward(h, ctx, cache)
        nxt = next_norm.row_params() if (next_norm is not None and hasattr(next_norm, "row_params")) else None
        if nxt is not None and nxt[0].numel() != W:
            nxt = None
        # (every reader of h is done when the kernel that overwrites it runs: the rows take its place)
        h2 = ws.tokens("block.normed", T, W, dt)
        s1 = self.tensors[self.names["mixer_scale"]] if self.layer_scale else None
        if self.feed_forward is not None:
            K.norm_add_norm(stream, a, s1, plain=True, next_norm=(*self.feed_forward_norm.row_params(), h2))
            s2 = self.tensors[self.names["feed_forward_scale"]] if self.layer_scale else None
            # a feed-forward whose last kernel can add to the stream itself (and leave the next norm's rows) does so
            takes = nxt is None or not nxt[2]  # (that kernel knows the norm without the mean taken off)
            if not (takes and self.feed_forward.forward_add(h2, ctx, stream, s2,
                                                            (nxt[0], nxt[1], h2) if nxt is not None else None)):
                f = self.feed_forward.forward(h2, ctx)
                K.norm_add_norm(stream, f, s2, plain=True, next_norm=(*nxt, h2) if nxt is not None else None)
        else:
            K.norm_add_norm(stream, a, s1, plain=True, next_norm=(*nxt, h2) if nxt is not None else None)
        if nxt is not None:
            ctx.prepared_norm = (next_norm, h2)
        ctx.stream_operand = None
        return None, stream
