"""Two attention mixers over a paged cache whose values are read out of what the keys already hold, both on the
general attention kernel with its further options (csrc/attention_generic.cu, csrc/attention_prep_shared.cu).

`kv_shared_attention`: grouped heads, q = W_q h, k = W_k h, and the VALUES ARE THE KEYS as projected (no value
projection).  Options, each a constructor argument:

* `whole_norm`: q and k pass an RMS norm over the whole projection (all heads at once, one weight per channel)
  before they are split into heads; the values stay the keys as projected, so the cache then holds normed keys
  and raw values in pages of their own.  Without it the cache holds the keys only and values are read from them.
* `slope_exponent` e: the score of (query at i, key at j) loses 2^(-e (h + 1) / H) * (i - j) for head h of H.
* `window` w: position i sees j with 0 <= i - j < w.  `pool` P (with a window): beside those, one mean key / value
  per block of P positions that lies wholly before the window (block b = positions bP .. bP + P - 1, seen when
  bP + P - 1 <= i - w); the means are formed from the pages as they hold the keys, when a block's last token
  arrives, and kept in a second cache with one entry per P tokens.  Tokens and blocks share one softmax.
* `gated`: the concatenated heads are multiplied by sigmoid(W_g h) in front of the output projection.

`latent_attention`: queries and keys / values through low-rank latents, run in the absorbed form.  With
c_q = RMSnorm(W_dq h), q = W_uq c_q (or, without a query latent, q = W_q h) laid out per head as
[dim unrotated | rot rotated], W_dkv h = [kv_rank | rot]
whose first part, RMS-normed, is the latent c and whose second part is ONE rotated key part shared by all heads,
per head k = [W_uk c | k_rot], v = W_uv c:

    score = (q_plain . W_uk c + q_rot . k_rot) * scale = ((W_uk^T q_plain) . c + q_rot . k_rot) * scale

so the cache holds one row [c | k_rot] per token (a single kv head), the query of head h becomes
[W_uk,h^T q_plain,h | q_rot,h], the values are the first kv_rank elements of the key rows, and the head's output
in latent space is taken through W_uv,h afterwards.  Rotation: neighbours (2i, 2i + 1), or the halves (i, i + dims / 2),
of the first `dims` rotated dimensions turn by position * theta^(-2i / dims), angles in 32-bit.  `gated`: the
concatenated heads (after W_uv) are multiplied by sigmoid(W_g h) in front of the output projection.
"""

from __future__ import annotations

import torch

from ..csrc import kernels
from .base import CacheNeed, Mixer, ParamDecl
from .linear import batched_matmul, linear
from .registry import build_position_encoding, register_mixer


class _ProjectsOutput:
    """What a mixer needs so that a caller can take over its output projection (see `ParallelMixers`): the rows in
    front of the projection go to `out` (a column range of wider rows, if the caller likes) times `out_scale`."""

    shared_o = None  # a caller's tensor for the output projection's weight (a column range of a wider matrix)

    def _make_o(self, make, name, shape):
        if self.shared_o is not None:
            if tuple(self.shared_o.shape) != tuple(shape):
                raise ValueError(f"the shared output projection has shape {tuple(self.shared_o.shape)}, not {shape}")
            return self.shared_o
        return make(name, ParamDecl(shape))


@register_mixer("kv_shared_attention")
class KVSharedAttention(Mixer, _ProjectsOutput):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, scale: float | None = None,
                 window: int | None = None, pool: int = 0, whole_norm: bool = False, norm_eps: float = 1e-6,
                 slope_exponent: float | None = None, gated: bool = False, names: dict | None = None):
        super().__init__()
        if min(hidden_size, num_heads, num_kv_heads, head_dim) <= 0 or num_heads % num_kv_heads:
            raise ValueError("sizes must be positive and num_heads a multiple of num_kv_heads")
        if head_dim > 512:
            raise ValueError(f"head_dim={head_dim}: the attention kernel takes up to 512")
        if window is not None and window <= 0:
            raise ValueError("window must be positive (None: every earlier token is seen)")
        if pool < 0 or (pool and window is None):
            raise ValueError("pooled blocks lie behind a window: pool needs one")
        if pool and slope_exponent is not None:
            raise ValueError("a pooled block has no distance: pool and slope_exponent exclude each other")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.scale = head_dim ** -0.5 if scale is None else float(scale)
        self.window, self.pool = window, int(pool)
        self.whole_norm, self.norm_eps = bool(whole_norm), float(norm_eps)
        self.slope_exponent = None if slope_exponent is None else float(slope_exponent)
        self.gated = bool(gated)
        n = dict(q="q_proj.weight", k="k_proj.weight", g="g_proj.weight", o="o_proj.weight", q_norm="q_norm",
                 k_norm="k_norm")
        n.update(names or {})
        self.names = n
        self.q_size = num_heads * head_dim
        self.kv_size = num_kv_heads * head_dim
        self.o_size = self.q_size  # the values are keys: as wide as they are
        self.slopes = None

    def param_decls(self):
        H, n = self.hidden_size, self.names
        d = {n["q"]: ParamDecl((self.q_size, H)), n["k"]: ParamDecl((self.kv_size, H)),
             n["o"]: ParamDecl((H, self.o_size))}
        if self.gated:
            d[n["g"]] = ParamDecl((self.o_size, H))
        if self.whole_norm:
            d[n["q_norm"]] = ParamDecl((self.q_size,), "norm")
            d[n["k_norm"]] = ParamDecl((self.kv_size,), "norm")
        return d

    def materialize(self, make):
        H, n, q, kv = self.hidden_size, self.names, self.q_size, self.kv_size
        # one product for q | k | output gate
        self.w_in = make("in_proj.weight", ParamDecl((q + kv + (self.o_size if self.gated else 0), H)))
        self.tensors[n["q"]] = self.w_in[:q]
        self.tensors[n["k"]] = self.w_in[q:q + kv]
        if self.gated:
            self.tensors[n["g"]] = self.w_in[q + kv:]
        self.tensors[n["o"]] = self._make_o(make, n["o"], (H, self.o_size))
        if self.whole_norm:
            self.tensors[n["q_norm"]] = make(n["q_norm"], ParamDecl((q,), "norm"))
            self.tensors[n["k_norm"]] = make(n["k_norm"], ParamDecl((kv,), "norm"))
        if self.slope_exponent is not None:
            h = torch.arange(1, self.num_heads + 1, dtype=torch.float64)
            s = torch.pow(torch.tensor(2.0, dtype=torch.float64), -self.slope_exponent * h / self.num_heads)
            self.slopes = s.to(torch.float32).to(self.w_in.device)

    # -- cache ------------------------------------------------------------
    def cache_need(self):
        # a block's tokens must still be in the pages when its last one arrives
        window = None if self.window is None else max(self.window, self.pool)
        return CacheNeed(self.num_kv_heads, self.head_dim, window, None, 0, values_in_keys=not self.whole_norm)

    def aux_cache_need(self):
        if not self.pool:
            return None
        return CacheNeed(self.num_kv_heads, self.head_dim, None, None, 0, values_in_keys=not self.whole_norm,
                         every=self.pool)

    def activation_elems(self):
        return self.q_size + self.kv_size + (2 if self.gated else 1) * self.o_size + self.hidden_size

    def graph_key_group(self):
        return (type(self), self.num_heads, self.num_kv_heads, self.head_dim, self.pool)

    def output_projection(self):
        return self.tensors[self.names["o"]], None

    def output_width(self) -> int:
        return self.o_size

    # -- one step ---------------------------------------------------------
    def forward(self, x, ctx, cache, project_output: bool = True, out=None, out_scale: float = 1.0):
        K = kernels()
        T = x.shape[0]
        ws, n, g = ctx.workspace, self.names, cache.group
        q, kv = self.q_size, self.kv_size
        if g is None or not cache.writes:
            raise RuntimeError("this attention keeps keys of its own: it was given no cache to write")
        qk = ws.tokens("kvs.in", T, self.w_in.shape[0], x.dtype)
        linear(x, self.w_in, qk)
        v_pages = cache.v_pages if self.whole_norm else None
        K.kv_shared_prepare(qk, q, kv, self.tensors[n["q_norm"]] if self.whole_norm else None,
                            self.tensors[n["k_norm"]] if self.whole_norm else None, self.norm_eps, g.slot_mapping,
                            cache.k_pages, v_pages)
        pooled = None
        if self.pool:
            aux = cache.aux
            if aux is None:
                raise RuntimeError("pooled blocks: the mixer was given no second cache")
            K.pool_blocks(ctx.positions, ctx.token_req, ctx.req_slots, g.block_table, g.page_size, cache.k_pages,
                          v_pages, aux.group.slot_mapping, aux.k_pages, aux.v_pages if self.whole_norm else None,
                          self.pool)
            pooled = (aux.k_pages, aux.v_pages if self.whole_norm else None, aux.group.block_table)
        attn = out if out is not None else ws.tokens("attn.out", T, self.o_size, x.dtype)
        K.windowed_attention(qk, attn, cache.k_pages, v_pages, g.block_table, g.req_slots, ctx.cu_q, g.kv_len,
                             ctx.token_req, self.num_heads, self.num_kv_heads, self.head_dim, self.head_dim,
                             g.page_size, self.window or 0, self.scale, slopes=self.slopes, pool=self.pool,
                             pooled=pooled, gate=qk[:, q + kv:] if self.gated else None, out_scale=out_scale,
                             num_requests=ctx.num_requests, workspace=ws)
        if not project_output:
            return attn
        res = ws.tokens("mixer.out", T, self.hidden_size, x.dtype)
        linear(attn, self.tensors[n["o"]], res)
        return res


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, value_dim: int,
                 q_rank: int | None, kv_rank: int, position, scale: float | None = None, window: int | None = None,
                 pool: int = 0, norm_eps: float = 1e-6, names: dict | None = None, gated: bool = False):
        """`head_dim`: the unrotated query / key size per head, `rot_dim` the rotated one; `position`: a
        `PositionSpec` of kind `rope_computed`, with `interleaved` or not (its `rotary_dim` <= `rot_dim` dimensions
        turn, the rest pass).  `q_rank` None: no query latent, one projection `q` gives the queries.  `window`,
        `pool`: as for `kv_shared_attention` (a pooled block's key row is the mean of the cached rows [c | k_rot],
        its value the mean latent).  `gated`: a sigmoid output gate `g` [heads * value_dim, hidden]."""
        super().__init__()
        if min(hidden_size, num_heads, head_dim, value_dim, kv_rank) <= 0 or rot_dim < 0 or (q_rank is not None and q_rank <= 0):
            raise ValueError("sizes must be positive")
        if kv_rank + rot_dim > 640 or kv_rank > 512:
            raise ValueError(f"kv_rank {kv_rank} + rot_dim {rot_dim}: the attention kernels take key rows up to 640 "
                             "and values up to 512")
        if window is not None and window <= 0:
            raise ValueError("window must be positive (None: every earlier token is seen)")
        if pool < 0 or (pool and window is None):
            raise ValueError("pooled blocks lie behind a window: pool needs one")
        self.hidden_size, self.num_heads, self.head_dim, self.rot_dim = hidden_size, num_heads, head_dim, rot_dim
        self.value_dim, self.q_rank, self.kv_rank = value_dim, q_rank, kv_rank
        self.gated = bool(gated)
        self.scale = (head_dim + rot_dim) ** -0.5 if scale is None else float(scale)
        self.window, self.pool, self.norm_eps = window, int(pool), float(norm_eps)
        self.position = build_position_encoding(position) if (position is not None and rot_dim) else None
        if self.position is not None:
            if not getattr(self.position, "computed", False):
                raise ValueError("latent attention takes a position encoding of kind 'rope_computed'")
            if self.position.rotary_dim > rot_dim:
                raise ValueError("more rotated dimensions than the rotated part has")
        n = dict(dq="q_a_proj.weight", dq_norm="q_a_norm", uq="q_b_proj.weight", q="q_proj.weight", dkv="kv_a_proj.weight",
                 dkv_norm="kv_a_norm", uk="k_b_proj.weight", uv="v_b_proj.weight", g="g_proj.weight", o="o_proj.weight")
        n.update(names or {})
        self.names = n
        self.key_row = kv_rank + rot_dim

    def param_decls(self):
        H, n, N = self.hidden_size, self.names, self.num_heads
        d = {
            n["dkv"]: ParamDecl((self.key_row, H)), n["dkv_norm"]: ParamDecl((self.kv_rank,), "norm"),
            n["uk"]: ParamDecl((N * self.head_dim, self.kv_rank)), n["uv"]: ParamDecl((N * self.value_dim, self.kv_rank)),
            n["o"]: ParamDecl((H, N * self.value_dim)),
        }
        if self.q_rank is None:
            d[n["q"]] = ParamDecl((N * (self.head_dim + self.rot_dim), H))
        else:
            d[n["dq"]] = ParamDecl((self.q_rank, H))
            d[n["dq_norm"]] = ParamDecl((self.q_rank,), "norm")
            d[n["uq"]] = ParamDecl((N * (self.head_dim + self.rot_dim), self.q_rank))
        if self.gated:
            d[n["g"]] = ParamDecl((N * self.value_dim, H))
        return d

    def materialize(self, make):
        n, N, H = self.names, self.num_heads, self.hidden_size
        self.w_in = None
        if self.q_rank is None:
            # one product for q | latent and rotated key part | output gate, all read from the mixer's input
            qw = N * (self.head_dim + self.rot_dim)
            self.w_in = make("in_proj.weight", ParamDecl((qw + self.key_row + (N * self.value_dim if self.gated else 0), H)))
            self.tensors[n["q"]] = self.w_in[:qw]
            self.tensors[n["dkv"]] = self.w_in[qw:qw + self.key_row]
            if self.gated:
                self.tensors[n["g"]] = self.w_in[qw + self.key_row:]
        for name, decl in self.param_decls().items():
            if name not in self.tensors:
                self.tensors[name] = make(name, decl)
        if self.position is not None:
            self.position.build_tables(self.tensors[n["dkv"]].device)

    def cache_need(self):
        window = None if self.window is None else max(self.window, self.pool)
        return CacheNeed(1, self.key_row, window, None, 0, values_in_keys=True)

    def aux_cache_need(self):
        return CacheNeed(1, self.key_row, None, None, 0, values_in_keys=True, every=self.pool) if self.pool else None

    def activation_elems(self):
        N = self.num_heads
        return ((self.q_rank or 0) + self.key_row + N * (self.head_dim + self.rot_dim) + N * self.kv_rank
                + N * self.key_row + N * self.kv_rank + (2 if self.gated else 1) * N * self.value_dim + self.hidden_size)

    def graph_key_group(self):
        return (type(self), self.num_heads, self.key_row, self.pool)

    def output_projection(self):
        return self.tensors[self.names["o"]], None

    def forward(self, x, ctx, cache):
        K = kernels()
        T = x.shape[0]
        ws, n, g, N = ctx.workspace, self.names, cache.group, self.num_heads
        d, r, R, dv = self.head_dim, self.rot_dim, self.kv_rank, self.value_dim
        if g is None or not cache.writes:
            raise RuntimeError("latent attention keeps a cache of its own: it was given none to write")
        dt = x.dtype
        gate = None
        if self.w_in is not None:
            qw = N * (d + r)
            both = ws.tokens("lat.in", T, self.w_in.shape[0], dt)
            linear(x, self.w_in, both)
            q_full, dkv = both[:, :qw], both[:, qw:qw + self.key_row]
            gate = both[:, qw + self.key_row:] if self.gated else None
        else:
            q_full = ws.tokens("lat.q", T, N * (d + r), dt)
            cq = ws.tokens("lat.cq", T, self.q_rank, dt)
            linear(x, self.tensors[n["dq"]], cq)
            K.add_rmsnorm(cq, None, self.tensors[n["dq_norm"]], self.norm_eps, cq)
            linear(cq, self.tensors[n["uq"]], q_full)
            dkv = ws.tokens("lat.dkv", T, self.key_row, dt)
            linear(x, self.tensors[n["dkv"]], dkv)
            if self.gated:
                gate = ws.tokens("lat.gate", T, N * dv, dt)
                linear(x, self.tensors[n["g"]], gate)
        # every head's unrotated query through its key up-projection, [heads, T, dim] x [heads, dim, rank], written
        # straight into the absorbed part of the query rows [T, heads, rank | rot]
        q_out = ws.tokens("lat.q_out", T, N * self.key_row, dt)
        batched_matmul(q_full.unflatten(1, (N, d + r))[:, :, :d].transpose(0, 1), self.tensors[n["uk"]].view(N, d, R),
                       q_out.view(T, N, self.key_row)[:, :, :R].transpose(0, 1))
        tables = self.position.tables() if self.position is not None else {}
        K.latent_prepare(q_full, None, dkv, q_out, N, d, r, R, self.position.rotary_dim if self.position else 0,
                         self.tensors[n["dkv_norm"]], self.norm_eps, tables.get("inv_freq"), ctx.positions,
                         g.slot_mapping, cache.k_pages, interleaved=bool(getattr(self.position, "interleaved", True)))
        pooled = None
        if self.pool:
            aux = cache.aux
            if aux is None:
                raise RuntimeError("pooled blocks: the mixer was given no second cache")
            K.pool_blocks(ctx.positions, ctx.token_req, ctx.req_slots, g.block_table, g.page_size, cache.k_pages, None,
                          aux.group.slot_mapping, aux.k_pages, None, self.pool)
            pooled = (aux.k_pages, None, aux.group.block_table)
        o_lat = ws.tokens("lat.o_lat", T, N * R, dt)
        K.windowed_attention(q_out, o_lat, cache.k_pages, None, g.block_table, g.req_slots, ctx.cu_q, g.kv_len,
                             ctx.token_req, N, 1, self.key_row, R, g.page_size, self.window or 0, self.scale,
                             pool=self.pool, pooled=pooled, num_requests=ctx.num_requests, workspace=ws)
        # each head's latent output through its value up-projection: [heads, T, rank] x [heads, rank, vdim]
        attn = ws.tokens("attn.out", T, N * dv, dt)
        batched_matmul(o_lat.view(T, N, R).transpose(0, 1), self.tensors[n["uv"]].view(N, dv, R).transpose(1, 2),
                       attn.view(T, N, dv).transpose(0, 1))
        if gate is not None:
            K.sigmoid_gate(attn, gate)
        out = ws.tokens("mixer.out", T, self.hidden_size, dt)
        linear(attn, self.tensors[n["o"]], out)
        return out
