"""A decoder assembled from a ModelSpec: embedding, blocks run in the order the
schedule gives, final norm, output head.  ullm/models/qwen3.py:228-255 and
:284-286 are the reference's fixed version of this loop.

The model owns no cache and no batch logic: `forward` receives the step's
context and one LayerCache per schedule entry.
"""

from __future__ import annotations

import torch

from ..config.specs import ModelSpec
from ..csrc import kernels
from .base import ParamDecl, Part
from .embedding import OutputHead, TokenEmbedding, TokenSideTable
from .registry import build_block, build_norm, build_position_encoding


class DecoderModel(Part):
    def __init__(self, spec: ModelSpec, untie_head: bool = False):
        super().__init__()
        spec.validate()
        self.spec = spec
        position = None
        if spec.embedding_position is not None:
            position = build_position_encoding(spec.embedding_position)
            if not getattr(position, "adds_to_embedding", lambda: False)():
                raise ValueError(f"position encoding {spec.embedding_position.kind!r} cannot be added to an embedding")
        self.embedding = TokenEmbedding(spec.vocab_size, spec.hidden_size, spec.embedding_scale, position,
                                        spec.embedding_param)
        if spec.stream_dtype not in ("engine", "float32"):
            raise ValueError(f"stream_dtype {spec.stream_dtype!r}: 'engine' or 'float32'")
        self.stream_f32 = spec.stream_dtype == "float32"
        if not self.stream_f32 and not self.embedding.plain():
            raise ValueError("a scaled embedding or an added position encoding needs stream_dtype='float32'")
        self.blocks = [build_block(ls) for ls in spec.layers]
        self.final_norm = build_norm(spec.final_norm)
        tied = spec.tie_embeddings and not untie_head
        self.head = OutputHead(spec.vocab_size, spec.hidden_size, self.embedding if tied else None, spec.head_param,
                               softcap=spec.logit_softcap)
        self.token_side = None
        if spec.token_side is not None:
            self.token_side = TokenSideTable(spec.vocab_size, spec.token_side.dim, spec.token_side.shares)
        self.schedule = list(spec.schedule)
        self._keeps_input = any(e.add_input or e.project_input for e in self.schedule)
        # one mixer of each group answers `graph_key` for all of its kind
        seen: dict = {}
        for e in self.schedule:
            m = self.blocks[e.layer].mixer
            seen.setdefault(m.graph_key_group(), m)
        self._graph_key_mixers = list(seen.values())
        self.dtype: torch.dtype | None = None
        self.device = None

    def subparts(self):
        s = {self.spec.embedding_name: self.embedding}
        for i, b in enumerate(self.blocks):
            s[self.spec.layer_name.format(i)] = b
        s[self.spec.final_norm_name] = self.final_norm
        s[self.spec.head_name] = self.head
        if self.token_side is not None:
            s[self.spec.token_side.name] = self.token_side
        return s

    def param_decls(self):
        d = {}
        if self.spec.pass_vectors is not None:
            name, rows = self.spec.pass_vectors
            d[name] = ParamDecl((rows, self.spec.hidden_size), "bias32")
        if self.spec.pass_projection is not None:
            d[self.spec.pass_projection] = ParamDecl((self.spec.hidden_size, 2 * self.spec.hidden_size))
        return d

    # -- what the cache manager needs to know ------------------------------
    def cache_needs(self):
        """Per schedule entry: (CacheNeed | None, StateNeed | None, cache_of, second CacheNeed | None)."""
        out = []
        for e in self.schedule:
            m = self.blocks[e.layer].mixer
            out.append((m.cache_need(), m.state_need(), e.cache_of, m.aux_cache_need()))
        return out

    def graph_key(self, ctx) -> tuple:
        """What of a decode step, beyond its padded size, decides the kernels its mixers launch."""
        return tuple(m.graph_key(ctx) for m in self._graph_key_mixers)

    # -- allocation ---------------------------------------------------------
    def allocate(self, device, dtype: torch.dtype) -> None:
        """Gives every declared parameter a tensor on `device`: matrices and
        biases in `dtype`, norm weights in float32."""
        self.dtype = dtype
        self.device = torch.device(device)

        def make(name, decl):
            dt = torch.float32 if decl.role in ("norm", "bias32") else dtype
            return torch.empty(decl.shape, dtype=dt, device=self.device)

        self.materialize_all(make)

    # -- one step -----------------------------------------------------------
    def forward_hidden(self, ctx, caches):
        """Runs the blocks over the step's tokens.  Returns (y, residual): what the last block left to be added
        (or None) and the residual stream, before the final norm."""
        T = ctx.num_tokens
        ctx.stream_operand = None
        ctx.token_side = self.token_side
        ctx.shared = {}  # what one execution leaves for later ones of the same step (first-layer values, say)
        if self.stream_f32:
            # the stream is 32-bit; its copy rounded to the engine's dtype is the first sub-layer's operand
            x = ctx.workspace.tokens("model.stream", T, self.spec.hidden_size, torch.float32)
            copy = None
            if self.dtype != torch.float32:
                copy = ctx.workspace.tokens("model.stream_copy", T, self.spec.hidden_size, self.dtype)
            self.embedding.forward_stream(ctx.token_ids, x, copy, ctx)
            ctx.stream_operand = copy if copy is not None else x
        else:
            x = ctx.workspace.tokens("model.hidden", T, self.spec.hidden_size, self.dtype)
            self.embedding.forward(ctx.token_ids, x, ctx)
        x0 = None
        if self._keeps_input:
            # the input as the embedding left it, for the executions that add it to the stream again
            x0 = ctx.workspace.tokens("model.input", T, self.spec.hidden_size, torch.float32)
            x0.copy_(x)
        residual = None
        n = len(self.schedule)
        for i, e in enumerate(self.schedule):
            block = self.blocks[e.layer]
            if e.project_input:
                self._project_stream(residual if residual is not None else x, x0, ctx)
            if e.add_input or e.add_vector is not None:
                self._add_to_stream(residual if residual is not None else x, x0 if e.add_input else None,
                                    e.add_vector, block, ctx)
            if block.takes_next_norm:
                # the norm that the next block applies first, if that block can start from what this one prepares
                # (not when something is added to the stream in between: that addition prepares it then)
                nxt = self.blocks[self.schedule[i + 1].layer] if i + 1 < n else None
                if nxt is not None and (self.schedule[i + 1].add_input or self.schedule[i + 1].add_vector is not None
                                        or self.schedule[i + 1].project_input):
                    nxt = None
                nxt_norm = nxt.mixer_norm if (nxt is not None and nxt.accepts_folded_norm()) else None
                x, residual = block.forward(x, residual, ctx, caches[i], next_norm=nxt_norm)
            else:
                x, residual = block.forward(x, residual, ctx, caches[i])
        ctx.folded_norm = None
        ctx.prepared_norm = None
        return x, residual

    def _project_stream(self, stream, x0, ctx) -> None:
        """stream <- P [stream | x0] with the model's pass projection P [hidden, 2 hidden]: the two 32-bit row sets
        side by side, rounded to the engine's dtype, are one product's operand; its 32-bit result is the new
        stream."""
        if stream is None or stream.dtype != torch.float32 or x0 is None:
            raise RuntimeError("a projection of the stream between layers needs a 32-bit stream and the kept input")
        T, H = stream.shape
        K = kernels()
        both = ctx.workspace.tokens("model.pass_in", T, 2 * H, self.dtype)
        K.concat_rows_f32(stream, x0, both)
        K.linear_f32_out(both, self.tensors[self.spec.pass_projection], stream)
        ctx.prepared_norm = None
        ctx.stream_operand = None

    def _add_to_stream(self, stream, rows, vector, block, ctx) -> None:
        """stream += rows (if given) + row `vector` of the pass vectors (if given), in this order, in 32-bit; the
        same kernel leaves the rows of the norm that `block` applies first, if it can start from them."""
        if stream is None or stream.dtype != torch.float32:
            raise RuntimeError("additions to the stream between layers need a 32-bit stream")
        vec = self.tensors[self.spec.pass_vectors[0]][vector] if vector is not None else None
        ctx.prepared_norm = None
        nxt = None
        if block.takes_next_norm and block.accepts_folded_norm() and hasattr(block.mixer_norm, "row_params"):
            params = block.mixer_norm.row_params()
            if params is not None and params[0].numel() == stream.shape[1]:
                h = ctx.workspace.tokens("block.normed", stream.shape[0], stream.shape[1], block.mixer.operand_dtype())
                nxt = (*params, h)
        kernels().norm_add_norm(stream, extra_rows=rows, extra_vec=vec, next_norm=nxt)
        if nxt is not None:
            ctx.prepared_norm = (block.mixer_norm, nxt[3])
        ctx.stream_operand = None

    def forward(self, ctx, caches):
        """Logits [len(ctx.logits_rows), vocab] float32 at the wanted rows."""
        y, residual = self.forward_hidden(ctx, caches)
        R = ctx.num_logits_rows
        if R == 0:
            return None
        K = kernels()
        H = self.spec.hidden_size
        ys = ctx.workspace.requests("head.y", R, H, self.dtype)
        if self.stream_f32:
            if y is not None and residual is not None:
                raise RuntimeError("a block of a 32-bit stream left something pending beside the stream")
            self.final_norm.forward_rows(residual if residual is not None else y, ctx.logits_rows, ys)
        elif y is None or residual is None:
            # nothing is pending beside the stream (a block that adds its own output), or there is no stream
            K.gather_rows(y if residual is None else residual, ctx.logits_rows, ys)
            self.final_norm.forward(ys, None, out=ys)
        else:
            rs = ctx.workspace.requests("head.res", R, H, self.dtype)
            K.gather_rows(y, ctx.logits_rows, ys)
            K.gather_rows(residual, ctx.logits_rows, rs)
            self.final_norm.forward(ys, rs, out=ys)
        logits = ctx.workspace.requests("head.logits", R, self.spec.vocab_size, torch.float32)
        self.head.forward(ys, logits)
        return logits
