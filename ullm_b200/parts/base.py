"""What every part is: an object built from sizes and constants alone, that
declares its parameters by name, receives tensors for them, and runs on a flat
batch of tokens.  No part knows which model it is in.

Interfaces (what a new part must have):

* every part: `param_decls() -> {name: ParamDecl}` and
  `materialize(make) -> None`, where `make(name, decl)` returns the tensor for a
  declared parameter; the part keeps what it needs and lists the tensors under
  their checkpoint names in `self.tensors`.
* Norm: `forward(x, residual=None, out=None) -> out`; with a residual the sum
  x + residual is formed in 32-bit, written back to `residual`, and normed.
* PositionEncoding: `tables() -> dict of device tensors` handed to the mixer's
  kernel, plus `rotary_dim`; or `transforms_qk() -> True` and `apply(q, k,
  positions)` for an encoding that is no rotation by tables.
* Mixer: `cache_need() -> CacheNeed | None`, `state_need() -> StateNeed | None`,
  `graph_key(ctx)` (what of a decode step changes its launches, default nothing),
  `forward(x[T, hidden], ctx, cache) -> [T, hidden]`; `cache` is the
  LayerCache of this execution (pages of its group + the group's step
  metadata, and its state rows if it asked for any).
* FeedForward: `forward(x[T, hidden], ctx) -> [T, hidden]`.
* Block: `forward(x, residual, ctx, cache) -> (x, residual)`.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch


@dataclass(frozen=True)
class ParamDecl:
    """A parameter as the checkpoint stores it.  `role` decides precision and
    random init: "matrix" (embedding and linear weights: engine dtype, N(0,
    std)), "bias" (engine dtype, N(0, std)), "norm" (always held in 32-bit,
    1 + N(0, norm_std)), "bias32" (a bias that enters 32-bit arithmetic: always
    held in 32-bit, N(0, std))."""

    shape: tuple[int, ...]
    role: str = "matrix"


@dataclass(frozen=True)
class CacheNeed:
    """Keys and values this mixer keeps per token: `num_kv_heads` x `head_dim`
    for K and `num_kv_heads` x `value_dim` for V (None: `head_dim`).  `window`:
    None keeps every token, w keeps the last w, and with `keep_first` also the
    first `keep_first` tokens of the request.  `values_in_keys`: there are no value
    pages (the mixer reads its values out of the key rows).  `every` n > 1: the
    cache holds one entry per n tokens (entry e is written when token (e + 1) n - 1
    arrives), all of them kept; its pages are counted in entries."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None
    value_dim: int | None = None
    keep_first: int = 0
    values_in_keys: bool = False
    every: int = 1

    @property
    def v_dim(self) -> int:
        if self.values_in_keys:
            return 0
        return self.head_dim if self.value_dim is None else self.value_dim


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size: one row of `shape` per live request."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


Maker = Callable[[str, ParamDecl], torch.Tensor]


class Part:
    def __init__(self) -> None:
        self.tensors: dict[str, torch.Tensor] = {}

    def param_decls(self) -> dict[str, ParamDecl]:
        return {}

    def materialize(self, make: Maker) -> None:
        for name, decl in self.param_decls().items():
            self.tensors[name] = make(name, decl)

    def subparts(self) -> dict[str, "Part"]:
        """Nested parts by tensor-name prefix."""
        return {}

    def activation_elems(self) -> int:
        """Elements per token that this part (with its sub-parts) keeps in the step's workspace while it
        runs; the engine sets that much memory aside before it sizes the cache pool.  A part that takes
        buffers from `ctx.workspace` says here how wide they are together."""
        return sum(p.activation_elems() for p in self.subparts().values())

    # -- walking a tree of parts ------------------------------------------
    def all_decls(self, prefix: str = "") -> dict[str, ParamDecl]:
        out = {prefix + n: d for n, d in self.param_decls().items()}
        for sub_prefix, sub in self.subparts().items():
            out.update(sub.all_decls(prefix + sub_prefix))
        return out

    def materialize_all(self, make: Maker, prefix: str = "") -> None:
        self.materialize(lambda n, d: make(prefix + n, d))
        for sub_prefix, sub in self.subparts().items():
            sub.materialize_all(make, prefix + sub_prefix)

    def all_tensors(self, prefix: str = "") -> dict[str, torch.Tensor]:
        out = {prefix + n: t for n, t in self.tensors.items()}
        for sub_prefix, sub in self.subparts().items():
            out.update(sub.all_tensors(prefix + sub_prefix))
        return out


class Norm(Part):
    def forward(self, x, residual=None, out=None):
        raise NotImplementedError

    def scale_add(self, a, stream, mult: float, copy=None):
        """stream (32-bit, in place) += mult * norm(a); `copy`, if given, receives the stream rounded to a's dtype.
        For arrangements that norm a sub-layer's output."""
        raise NotImplementedError

    def forward_rows(self, stream, rows, out):
        """out[r] = norm(stream[rows[r]]) for a 32-bit stream (`rows` None: every row), rounded to out's dtype."""
        raise NotImplementedError

    def row_params(self):
        """(weight, eps, centred) if this norm is w * (x - mean) / sqrt(variance + eps) over the whole row (centred)
        or w * x / sqrt(mean(x^2) + eps) (not centred), which a block may then hand to a kernel that norms a
        sub-layer's output, adds it to the stream and applies the next norm at once; None otherwise."""
        return None

    def rms_params(self):
        """(weight, eps) if this norm is a plain RMSNorm over the whole row, which a block may then fold into a
        fused kernel; None otherwise."""
        return None


class PositionEncoding(Part):
    """Two kinds.  A rotation by per-position tables hands `tables()` (`cos` / `sin` rows of `rotary_dim / 2`
    floats per position) to the mixer's kernels, which rotate in 32-bit registers.  Any other encoding that acts
    on queries and keys answers True from `transforms_qk()` and does its work in `apply`, with device code of
    its own; the mixer then norms q and k first and stores the keys afterwards.  (An encoding that biases the
    SCORES by both positions would need an argument of the attention kernels; there is none yet.)"""

    rotary_dim: int = 0

    def build_tables(self, device) -> None:
        """Called once, when the mixer's parameters exist: put what the encoding needs on `device`."""

    def tables(self) -> dict[str, torch.Tensor]:
        return {}

    def transforms_qk(self) -> bool:
        return False

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        """Changes this step's queries q [T, heads, head_dim] and keys k [T, kv heads, head_dim] in place
        (views of the projection's output); positions [T] int32 on the device."""
        raise NotImplementedError


class Mixer(Part):
    def cache_need(self) -> CacheNeed | None:
        return None

    def state_need(self) -> StateNeed | None:
        return None

    def aux_cache_need(self) -> CacheNeed | None:
        """A second cache of the same execution (pooled entries beside the tokens' pages, say); the mixer finds
        it as `cache.aux` (pages, the group's step data)."""
        return None

    def graph_key(self, ctx):
        """What about a decode step, beyond its padded batch size, changes the kernels this mixer launches or
        their grids (a mixer that picks a kernel by how unequal the requests' lengths are, say).  A recorded
        CUDA graph is replayed only for steps with the same key.  Hashable; () when nothing does."""
        return ()

    def graph_key_group(self):
        """Mixers with equal groups give equal graph keys for the same step (one of them is asked)."""
        return type(self)

    def takes_input_norm(self) -> bool:
        """True when `forward(..., input_norm=(sq, cols, eps))` is understood: x is then r * w (the norm weight
        already applied) and the mixer's first product multiplies its sums by the rows' 1 / rms, computed from the
        sums of squares `sq` (see `Kernels.stream_linear`).  Only asked for in small decode steps."""
        return False

    def output_projection(self):
        """(weight [hidden, width], bias or None) if the mixer ends in a plain linear map and can also stop in
        front of it (`forward(..., project_output=False)` then returns its [T, width] input); None otherwise.
        A block may fold that product into a fused kernel."""
        return None

    def operand_dtype(self):
        """The dtype of the rows this mixer's `forward` takes (that of its first matrix)."""
        for t in self.all_tensors().values():
            if t.dim() >= 2:
                return t.dtype
        raise RuntimeError("this mixer has no matrix to read its operand's dtype from")

    def forward(self, x, ctx, cache):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, ctx):
        raise NotImplementedError

    def forward_add(self, x, ctx, stream, scale=None, next_norm=None) -> bool:
        """Optional: stream (32-bit, in place) += scale * forward(x) in the part's own last kernel (`scale` a
        32-bit vector per channel or None), which also leaves the RMS norm `next_norm` = (weight, eps, out) of the
        updated rows.  False (the default): the caller adds `forward(x)` itself."""
        return False

    def gated_weights(self):
        """(w_gate_up [2 I, hidden], w_down [hidden, I], activation code) if this is a bias-free gated
        feed-forward down(act(gate(x)) * up(x)) that a block may fold into a fused kernel; None otherwise."""
        return None


class Block(Part):
    takes_next_norm = False  # True: `forward` has a `next_norm=` argument (see PreNormResidualBlock)

    def accepts_folded_norm(self) -> bool:
        return False

    def forward(self, x, residual, ctx, cache):
        raise NotImplementedError
