"""Grouped-query attention over a paged cache: qkv projection, optional
per-head q/k norm, position rotation, the write of this step's keys and values
into the pages, attention over the pages, output projection.

ullm/models/qwen3.py:113-130 gives the order (projection, q/k norm per head
over head_dim with one weight shared by all heads, rotation, attention, output
projection); ullm/models/qwen3.py:81 the scale; query head h reads kv head
h // (num_heads / num_kv_heads).  The three projections are one matrix with
rows q | k | v, as ullm/layers/linear.py:381-389 lays them out; the checkpoint's
q_proj / k_proj / v_proj tensors are row ranges of it.
"""

from __future__ import annotations

import torch

from ..csrc import check_attention_sizes, kernels
from .base import CacheNeed, Mixer, ParamDecl, StateNeed
from .linear import linear
from .registry import build_norm, build_position_encoding, register_mixer


def is_ragged(batch: int, max_kv: int, sum_kv: int) -> bool:
    """A decode batch whose longest request, times the batch, is more than 1.5 times all the keys there are:
    splitting every request alike would then leave most blocks waiting for the long one (measured: the
    batch-balanced attention kernel wins from about this ratio on, and loses about 5 % on even batches)."""
    return batch > 1 and 2 * batch * max_kv > 3 * sum_kv


@register_mixer("paged_attention")
class PagedAttention(Mixer):
    def __init__(
        self,
        hidden_size: int,
        num_heads: int,
        num_kv_heads: int,
        head_dim: int,
        qkv_bias: bool = False,
        qk_norm=None,
        position=None,
        window: int | None = None,
        scale: float | None = None,
        value_dim: int | None = None,
        keep_first: int = 0,
        own_kv: bool = True,
        names: dict | None = None,
        conv_taps: int = 0,
        score_cap: float | None = None,
        talking_heads: bool = False,
        value_mix: str | None = None,
        unit_norm_after_rotation: bool = False,
        norm_eps: float = 0.0,
        whole_norm: bool = False,
        value_unit_norm: bool = False,
        head_temperature: bool = False,
    ):
        """`value_dim`: head size of the values and of the output (default: `head_dim`).  `window` with
        `keep_first`: position i sees j <= i if i - j < window or j < keep_first.  `own_kv` False: the mixer has
        no key / value projections (nor a key norm); it reads the cache of the execution the schedule names
        (`ScheduleEntry.cache_of`) with queries, mask and scale of its own.  `names`: the checkpoint's names of
        q, k, v, o, q_norm, k_norm behind the mixer's prefix (defaults: `q_proj.weight`, ..., `q_norm.`).

        Further options, all on the general path (csrc/attention_prep.cu, then the tensor-core attention kernels
        where dtype and head sizes allow, else csrc/attention_generic.cu) in prompt and decode steps alike.
        `conv_taps` > 0: every channel of q, k and v passes a causal filter over time of that many taps before
        anything else happens to it (filters `q_conv`, `k_conv`, `v_conv` [channels, taps]); a request keeps its
        last taps - 1 projected rows as state.  `score_cap` c: score <-
        c tanh(score / c) after the scale.  `talking_heads`: the softmax weights are mixed across heads by the
        matrix `talk` [heads, heads], w'_h = sum_g talk[h, g] w_g, and the output of head h is w'_h times the
        values of the kv head that h belongs to.  `value_mix`: "first": this execution leaves its values of the step's tokens for later ones;
        "mix": v <- (1 - lambda) v + lambda v_first with the scalar `vmix` (what goes to the cache is the blend); both kinds
        declare the scalar.  `unit_norm_after_rotation`: q and k are divided by their root mean square over the
        head (eps `norm_eps`, no weight) behind the rotation.  A position of kind `rope_computed` (angles computed
        in the kernel, optional frequency scaling) also takes this path.

        Three more, prepared by csrc/attention_prep_shared.cu (`qkv_rows_prepare`) in front of the same attention
        kernels.  `whole_norm`: the q/k norm (`qk_norm`) runs over the WHOLE projection, all heads at once, with a
        weight per channel (`q_norm` [heads * head_dim], `k_norm` [kv heads * head_dim]), before the rotation.
        `value_unit_norm`: every head's value is divided by its root mean square (eps `norm_eps`, no weight); the
        cache holds it so.  `head_temperature`: the scores of head h are multiplied by the learned number `temp`[h]
        (it is folded into the prepared queries in 32-bit).  With any of them a `rope_computed` position may say
        `interleaved=True` (neighbouring dimensions turn together)."""
        super().__init__()
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads={num_heads} is no multiple of num_kv_heads={num_kv_heads}")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.qkv_bias = qkv_bias
        self.window = window
        self.scale = head_dim ** -0.5 if scale is None else scale
        self.value_dim = head_dim if value_dim is None else value_dim
        self.keep_first = int(keep_first)
        self.own_kv = bool(own_kv)
        if self.keep_first < 0 or self.value_dim <= 0:
            raise ValueError("keep_first must not be negative and value_dim must be positive")
        self.conv_taps = int(conv_taps)
        self.score_cap = float(score_cap) if score_cap else None
        self.talking_heads = bool(talking_heads)
        self.value_mix = value_mix
        self.unit_norm_after_rotation = bool(unit_norm_after_rotation)
        self.norm_eps = float(norm_eps)
        self.whole_norm = bool(whole_norm)
        self.value_unit_norm = bool(value_unit_norm)
        self.head_temperature = bool(head_temperature)
        # the form that `qkv_rows_prepare` prepares
        self.rows_form = self.whole_norm or self.value_unit_norm or self.head_temperature
        if self.rows_form and (conv_taps or value_mix or unit_norm_after_rotation or talking_heads or qkv_bias
                               or not own_kv or keep_first):
            raise ValueError("whole_norm / value_unit_norm / head_temperature do not combine with the convolution, value "
                             "mixing, the norm behind the rotation, mixed heads, biases, kept tokens or borrowed keys")
        if self.whole_norm and qk_norm is None:
            raise ValueError("whole_norm needs the norm's spec (qk_norm)")
        if self.conv_taps < 0 or self.conv_taps > 32:
            raise ValueError(f"conv_taps={conv_taps}: the convolution kernel takes 1 to 32 taps (0: none)")
        if self.score_cap is not None and self.score_cap <= 0:
            raise ValueError("score_cap must be positive")
        if value_mix not in (None, "first", "mix"):
            raise ValueError(f"value_mix={value_mix!r}: None, 'first' or 'mix'")
        if not self.own_kv and (self.conv_taps or value_mix):
            raise ValueError("a mixer without key / value projections has no values to convolve or to mix")
        n = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", o="o_proj.weight", q_bias="q_proj.bias",
                 k_bias="k_proj.bias", v_bias="v_proj.bias", q_norm="q_norm.", k_norm="k_norm.",
                 q_conv="q_proj.conv", k_conv="k_proj.conv", v_conv="v_proj.conv", talk="talk", vmix="vmix",
                 temp="temp")
        n.update(names or {})
        self.names = n
        self.q_size = num_heads * head_dim
        self.kv_size = num_kv_heads * head_dim
        self.v_size = num_kv_heads * self.value_dim
        self.o_size = num_heads * self.value_dim
        if self.whole_norm:
            from dataclasses import replace

            self.q_norm = build_norm(replace(qk_norm, size=self.q_size))
            self.k_norm = build_norm(replace(qk_norm, size=self.kv_size))
        else:
            self.q_norm = build_norm(qk_norm) if qk_norm is not None else None
            self.k_norm = build_norm(qk_norm) if (qk_norm is not None and self.own_kv) else None
        if self.whole_norm and self.value_unit_norm and self.q_norm.eps != self.norm_eps:
            raise ValueError("the whole-projection norm and the values' unit norm share one eps (qk_norm.eps = norm_eps)")
        if self.rows_form and not self.whole_norm and qk_norm is not None:
            raise ValueError("value_unit_norm / head_temperature take the q/k norm over the whole projection or none")
        self.position = build_position_encoding(position) if position is not None else None
        if getattr(self.position, "interleaved", False) and not self.rows_form:
            raise ValueError("a rotation of neighbouring dimensions needs whole_norm, value_unit_norm or head_temperature")
        self.general = bool(self.conv_taps or self.score_cap or self.talking_heads or value_mix or self.rows_form
                            or self.unit_norm_after_rotation or getattr(self.position, "computed", False))
        if self.general and self.position is not None and not getattr(self.position, "computed", False):
            raise ValueError("these attention options take a position encoding of kind 'rope_computed' (or none)")
        check_attention_sizes(num_heads, num_kv_heads, head_dim, self.position.rotary_dim if self.position else 0)

    # -- parameters -------------------------------------------------------
    def param_decls(self):
        H, n = self.hidden_size, self.names
        d = {n["q"]: ParamDecl((self.q_size, H)), n["o"]: ParamDecl((H, self.o_size))}
        if self.own_kv:
            d[n["k"]] = ParamDecl((self.kv_size, H))
            d[n["v"]] = ParamDecl((self.v_size, H))
        if self.qkv_bias:
            d[n["q_bias"]] = ParamDecl((self.q_size,), "bias")
            if self.own_kv:
                d[n["k_bias"]] = ParamDecl((self.kv_size,), "bias")
                d[n["v_bias"]] = ParamDecl((self.v_size,), "bias")
        if self.conv_taps:
            d[n["q_conv"]] = ParamDecl((self.q_size, self.conv_taps))
            d[n["k_conv"]] = ParamDecl((self.kv_size, self.conv_taps))
            d[n["v_conv"]] = ParamDecl((self.v_size, self.conv_taps))
        if self.talking_heads:
            d[n["talk"]] = ParamDecl((self.num_heads, self.num_heads), "bias32")
        if self.value_mix:
            d[n["vmix"]] = ParamDecl((), "bias32")
        if self.head_temperature:
            d[n["temp"]] = ParamDecl((self.num_heads,), "norm")
        return d

    def subparts(self):
        s = {}
        if self.q_norm is not None:
            s[self.names["q_norm"]] = self.q_norm
        if self.k_norm is not None:
            s[self.names["k_norm"]] = self.k_norm
        return s

    def materialize(self, make):
        H, q, kv, n = self.hidden_size, self.q_size, self.kv_size, self.names
        rows = q + ((kv + self.v_size) if self.own_kv else 0)
        self.w_qkv = make("qkv_proj.weight", ParamDecl((rows, H)))
        self.tensors[n["q"]] = self.w_qkv[:q]
        if self.own_kv:
            self.tensors[n["k"]] = self.w_qkv[q:q + kv]
            self.tensors[n["v"]] = self.w_qkv[q + kv:]
        self.tensors[n["o"]] = make("o_proj.weight", ParamDecl((H, self.o_size)))
        self.b_qkv = None
        if self.qkv_bias:
            self.b_qkv = make("qkv_proj.bias", ParamDecl((rows,), "bias"))
            self.tensors[n["q_bias"]] = self.b_qkv[:q]
            if self.own_kv:
                self.tensors[n["k_bias"]] = self.b_qkv[q:q + kv]
                self.tensors[n["v_bias"]] = self.b_qkv[q + kv:]
        self.w_conv = None
        if self.conv_taps:
            # the three filters one after the other, as the projection's rows are
            self.w_conv = make("qkv_proj.conv", ParamDecl((rows, self.conv_taps)))
            self.tensors[n["q_conv"]] = self.w_conv[:q]
            self.tensors[n["k_conv"]] = self.w_conv[q:q + kv]
            self.tensors[n["v_conv"]] = self.w_conv[q + kv:]
        if self.talking_heads:
            self.tensors[n["talk"]] = make(n["talk"], ParamDecl((self.num_heads, self.num_heads), "bias32"))
        if self.value_mix:
            self.tensors[n["vmix"]] = make(n["vmix"], ParamDecl((), "bias32"))
        if self.head_temperature:
            self.tensors[n["temp"]] = make(n["temp"], ParamDecl((self.num_heads,), "norm"))
        if self.position is not None:
            self.position.build_tables(self.w_qkv.device)

    # -- cache ------------------------------------------------------------
    def cache_need(self):
        return CacheNeed(self.num_kv_heads, self.head_dim, self.window,
                         None if self.value_dim == self.head_dim else self.value_dim, self.keep_first if self.window else 0)

    def state_need(self):
        """The convolution's memory: the last taps - 1 projected rows (q | k | v) of the request, 32-bit."""
        if self.conv_taps > 1:
            return StateNeed(((self.conv_taps - 1) * (self.q_size + self.kv_size + self.v_size),), torch.float32)
        return None

    def activation_elems(self):
        # qkv, the attention's output, the projected output; on the general path also the prepared queries, the
        # first layer's values, and with mixed heads every head's weights on every kv head's values in 32-bit
        n = self.q_size + self.kv_size + self.v_size + self.o_size + self.hidden_size
        if self.general:
            n += self.q_size + self.v_size
            if self.talking_heads:
                n += 2 * self.num_kv_heads * self.o_size
        return n

    # -- which kernels a decode step takes ---------------------------------
    def graph_key(self, ctx):
        return ("ragged",) if self._ragged(ctx) else ()

    def graph_key_group(self):
        return (type(self), self.num_heads, self.num_kv_heads, self.head_dim)

    @staticmethod
    def _ragged(ctx) -> bool:
        return bool(ctx.decode_only and is_ragged(ctx.num_live_requests, ctx.max_kv_len, ctx.sum_kv_len))

    def output_projection(self):
        return self.tensors[self.names["o"]], None

    def takes_input_norm(self):
        return not self.general

    # -- the general path ----------------------------------------------------
    def _forward_general(self, x, ctx, cache, project_output: bool):
        """Projection, then csrc/attention_prep.cu (convolution, rotation, norms, value mixing, cache stores), the
        general attention kernel (cap, window, kept tokens), and the mixing of heads if there is any."""
        K = kernels()
        T = x.shape[0]
        ws = ctx.workspace
        if not self.own_kv:
            raise NotImplementedError("borrowed keys and values beside these attention options")
        qkv = ws.tokens("attn.qkv", T, self.w_qkv.shape[0], x.dtype)
        linear(x, self.w_qkv, qkv, self.b_qkv)
        g = cache.group
        q = ws.tokens("attn.q", T, self.q_size, x.dtype)
        tables = self.position.tables() if self.position is not None else {}
        rotary_dim = self.position.rotary_dim if self.position is not None else 0
        v_first, mode = None, 0
        if self.value_mix == "first":
            v_first = ws.tokens("attn.v_first", T, self.v_size, x.dtype)
            ctx.shared["attn.v_first"] = v_first
            mode = 1
        elif self.value_mix == "mix":
            v_first = ctx.shared.get("attn.v_first")
            if v_first is None or v_first.shape != (T, self.v_size):
                raise RuntimeError("value mixing: no earlier execution of this step left values of this width")
            mode = 2
        state = cache.state if self.conv_taps > 1 else None
        if self.conv_taps > 1 and state is None:
            raise RuntimeError("the attention's convolution was given no state rows")
        if self.rows_form:
            K.qkv_rows_prepare(
                qkv, q, self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim, ctx.positions,
                g.slot_mapping if cache.writes else None, cache.k_pages, cache.v_pages,
                q_w=self.q_norm.weight if self.whole_norm else None, k_w=self.k_norm.weight if self.whole_norm else None,
                eps=self.q_norm.eps if self.whole_norm else self.norm_eps, inv_freq=tables.get("inv_freq"),
                rotary_dim=rotary_dim, interleaved=bool(getattr(self.position, "interleaved", False)),
                q_head_scale=self.tensors[self.names["temp"]] if self.head_temperature else None,
                value_unit_norm=self.value_unit_norm)
            return self._attend(q, x, ctx, cache, project_output)
        K.qkv_prepare(
            qkv, q, self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim, ctx.positions,
            g.slot_mapping if cache.writes else None, cache.k_pages, cache.v_pages,
            conv_w=self.w_conv, taps=self.conv_taps, conv_state=state, cu_q=ctx.cu_q, token_req=ctx.token_req,
            req_slots=ctx.req_slots, inv_freq=tables.get("inv_freq"), rotary_dim=rotary_dim,
            q_w=self.q_norm.weight if self.q_norm is not None else None,
            k_w=self.k_norm.weight if self.k_norm is not None else None, norm_first=self.q_norm is not None,
            norm_last=self.unit_norm_after_rotation,
            eps=self.q_norm.eps if self.q_norm is not None else self.norm_eps,
            vmix_mode=mode, vmix_lambda=self.tensors[self.names["vmix"]] if mode == 2 else None, v_first=v_first)
        if state is not None:
            K.conv_state_update(qkv, self.conv_taps, state, ctx.cu_q, ctx.token_req, ctx.req_slots, ctx.num_requests)
        return self._attend(q, x, ctx, cache, project_output)

    def _attend(self, q, x, ctx, cache, project_output: bool):
        """The prepared queries over the pages, then the mixing of heads (if any) and the output projection."""
        K = kernels()
        T = x.shape[0]
        ws, g = ctx.workspace, cache.group
        attn = ws.tokens("attn.out", T, self.o_size, x.dtype)
        parts = None
        if self.talking_heads:
            parts = ws.tokens("attn.parts", T, self.num_heads * self.num_kv_heads * self.value_dim, torch.float32)
        if self.rows_form and (self.value_dim != self.head_dim or self.head_dim not in (64, 128)):
            # head sizes the kernels below take only in their general form: the windowed kernel runs multiples of 16
            # on the tensor cores (and falls back to the general kernel itself)
            K.windowed_attention(q, attn, cache.k_pages, cache.v_pages, g.block_table, g.req_slots, ctx.cu_q, g.kv_len,
                                 ctx.token_req, self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim,
                                 g.page_size, self.window or 0, self.scale, num_requests=ctx.num_requests, workspace=ws)
            if not project_output:
                return attn
            out = ws.tokens("mixer.out", T, self.hidden_size, x.dtype)
            linear(attn, self.tensors[self.names["o"]], out)
            return out
        K.paged_attention(
            q, attn, cache.k_pages, cache.v_pages, g.block_table, g.req_slots, ctx.cu_q, g.kv_len, ctx.token_req,
            self.num_heads, self.num_kv_heads, self.head_dim, g.page_size, self.window or 0, self.scale, ctx,
            v_dim=self.value_dim, keep_first=self.keep_first if self.window else 0, softcap=self.score_cap or 0.0,
            parts=parts, general=True)
        if parts is not None:
            K.mix_heads(parts, self.tensors[self.names["talk"]], attn, self.num_heads, self.num_kv_heads, self.value_dim)
        if not project_output:
            return attn
        out = ws.tokens("mixer.out", T, self.hidden_size, x.dtype)
        linear(attn, self.tensors[self.names["o"]], out)
        return out

    # -- one step ---------------------------------------------------------
    def forward(self, x, ctx, cache, project_output: bool = True, input_norm=None):
        if self.general:
            if input_norm is not None:
                raise RuntimeError("a folded norm was handed to an attention that does not take one")
            return self._forward_general(x, ctx, cache, project_output)
        K = kernels()
        T = x.shape[0]
        ragged = self._ragged(ctx)
        if not self.own_kv and cache.writes:
            raise RuntimeError("a mixer without key / value projections must read another execution's cache "
                               "(ScheduleEntry.cache_of)")
        plain = self.own_kv and self.value_dim == self.head_dim and self.keep_first == 0
        qkv = ctx.workspace.tokens("attn.qkv", T, self.w_qkv.shape[0], x.dtype)
        if input_norm is not None:
            # x is r * w: the projection multiplies its sums by the rows' 1 / rms (a norm folded in front of it)
            if not K.stream_linear(x, self.w_qkv, qkv, self.b_qkv, norm_in_front=input_norm):
                raise RuntimeError("the projection with a folded norm was refused")
        else:
            linear(x, self.w_qkv, qkv, self.b_qkv)
        g = cache.group
        tables = self.position.tables() if self.position is not None else {}
        q_w = self.q_norm.weight if self.q_norm is not None else None
        k_w = self.k_norm.weight if self.k_norm is not None else None
        eps = self.q_norm.eps if self.q_norm is not None else 0.0
        rotary_dim = self.position.rotary_dim if self.position is not None else 0
        slot_mapping = g.slot_mapping if cache.writes else None
        fuse = None
        if not plain:
            # values of a head size of their own, kept first positions or borrowed keys and values: the general
            # kernels (norm / rotation / page write, then attention), in prompt and decode steps alike
            if self.position is not None and self.position.transforms_qk():
                raise NotImplementedError("a position encoding with code of its own beside these attention options")
            K.qk_norm_rope_store(
                qkv, self.num_heads, self.num_kv_heads, self.head_dim, q_w, k_w, eps, tables.get("cos"),
                tables.get("sin"), rotary_dim, ctx.positions, slot_mapping, cache.k_pages, cache.v_pages,
                v_dim=self.value_dim, kv_in_row=self.own_kv,
            )
        elif self.position is not None and self.position.transforms_qk():
            # an encoding with code of its own: norm q and k, let it change them, then store the keys and values
            if q_w is not None or k_w is not None:
                K.qk_norm_in_place(qkv, self.num_heads, self.num_kv_heads, self.head_dim, q_w, k_w, eps)
            self.position.apply(qkv[:, :self.q_size].view(T, self.num_heads, self.head_dim),
                                qkv[:, self.q_size:self.q_size + self.kv_size].view(T, self.num_kv_heads, self.head_dim),
                                ctx.positions)
            if slot_mapping is not None:
                K.qk_norm_rope_store(qkv, self.num_heads, self.num_kv_heads, self.head_dim, None, None, 0.0, None, None, 0,
                                     ctx.positions, slot_mapping, cache.k_pages, cache.v_pages)
        elif K.decode_fusion_applies(ctx, qkv, self.num_heads, self.num_kv_heads, self.head_dim, g.page_size, rotary_dim,
                                     tables.get("cos"), ragged):
            # a decode step: the attention kernel norms and rotates q and k and writes k and v to their pages itself
            fuse = dict(q_w=q_w, k_w=k_w, eps=eps, cos=tables["cos"], sin=tables["sin"], positions=ctx.positions,
                        slot_mapping=slot_mapping)
        else:
            K.qk_norm_rope_store(
                qkv, self.num_heads, self.num_kv_heads, self.head_dim, q_w, k_w, eps, tables.get("cos"),
                tables.get("sin"), rotary_dim, ctx.positions, slot_mapping, cache.k_pages, cache.v_pages,
            )
        attn = ctx.workspace.tokens("attn.out", T, self.o_size, x.dtype)
        K.paged_attention(
            qkv, attn, cache.k_pages, cache.v_pages, g.block_table, g.req_slots, ctx.cu_q, g.kv_len,
            ctx.token_req,
            self.num_heads, self.num_kv_heads, self.head_dim, g.page_size,
            self.window or 0, self.scale, ctx, ragged=ragged, **({"fuse": fuse} if fuse is not None else {}),
            **({} if plain else {"v_dim": self.value_dim, "keep_first": self.keep_first if self.window else 0}),
        )
        if not project_output:
            return attn  # (the caller multiplies by `output_projection()` itself)
        out = ctx.workspace.tokens("mixer.out", T, self.hidden_size, x.dtype)
        linear(attn, self.tensors[self.names["o"]], out)
        return out
