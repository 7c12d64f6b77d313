"""Architecture-neutral description of a decoder: what each layer is made of
and in which order layers run.  An architecture's config (see qwen3.py) is
translated into these; the parts are built from these and never see the
architecture's own config.

Every size and constant of a part is a field here.  Layers may differ from one
another: `ModelSpec.layers` is a list, not a count.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class NormSpec:
    """`args`: further keyword arguments of the norm's constructor (the name its weight has in the checkpoint,
    say)."""

    kind: str  # key in parts.registry.NORMS
    size: int
    eps: float
    args: dict[str, Any] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class PositionSpec:
    """`args`: further keyword arguments of the encoding's constructor (a scaling factor, say), for kinds
    that need more than the three constants every rotary table has."""

    kind: str  # key in parts.registry.POSITION_ENCODINGS ("rope", "none", ...)
    rotary_dim: int = 0
    theta: float = 10000.0
    max_positions: int = 0
    args: dict[str, Any] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class MixerSpec:
    """`kind` chooses the class from parts.registry.MIXERS; `args` are its
    constructor's keyword arguments (sizes, constants, nested specs)."""

    kind: str
    args: dict[str, Any] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str  # key in parts.registry.FEED_FORWARDS
    args: dict[str, Any] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class LayerSpec:
    """One block: which arrangement (`block`, key in parts.registry.BLOCKS)
    of which mixer, feed-forward and norms.  `names` maps the block's sub-part
    roles to the tensor-name prefixes the checkpoint uses for them."""

    block: str
    mixer: MixerSpec
    feed_forward: FeedForwardSpec | None  # None: the layer has no feed-forward (and no norm for it)
    mixer_norm: NormSpec
    feed_forward_norm: NormSpec | None
    names: dict[str, str] = field(default_factory=dict, hash=False, compare=False)
    # further keyword arguments of the block's constructor (a residual multiplier, say)
    block_args: dict[str, Any] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.  `layer` indexes ModelSpec.layers (a layer may
    be named by several entries: its weights are shared, each execution has a
    cache of its own).  `cache_of`, if set, is the index of an EARLIER schedule
    entry whose cache this execution reads instead of writing one of its own.
    What is added to the residual stream right before this execution (a pass of a loop over layers starts here,
    say): `add_input` the model's input as the embedding left it, `add_vector` row of the model's table of pass
    vectors (`ModelSpec.pass_vectors`); input first, then the vector.  `project_input`: right before this execution
    the stream is REPLACED by a projection of [stream | the model's input as the embedding left it] with the
    model's pass projection (`ModelSpec.pass_projection`, [hidden, 2 hidden]); before any addition."""

    layer: int
    cache_of: int | None = None
    add_input: bool = False
    add_vector: int | None = None
    project_input: bool = False


@dataclass(frozen=True)
class TokenSideSpec:
    """A second embedding table [vocab, shares * dim] of which every layer reads a share of `dim` columns of its
    tokens' rows (a per-layer token input).  `name`: the table's tensor name."""

    name: str
    dim: int
    shares: int


@dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: list[LayerSpec]
    schedule: list[ScheduleEntry]
    final_norm: NormSpec
    tie_embeddings: bool
    max_positions: int
    dtype: str  # the checkpoint's own dtype ("bfloat16", "float32", "float16")
    embedding_name: str = "model.embed_tokens."
    layer_name: str = "model.layers.{}."
    final_norm_name: str = "model.norm."
    head_name: str = "lm_head."
    eos_token_id: int | None = None
    # the name of the table inside the embedding's and the head's prefix
    embedding_param: str = "weight"
    head_param: str = "weight"
    # x0 = table[id] * embedding_scale (+ an absolute position encoding that is added to the embedding)
    embedding_scale: float = 1.0
    embedding_position: PositionSpec | None = None
    # "engine": the residual stream has the engine's dtype; "float32": it is kept in 32-bit whatever the engine's
    # dtype (the blocks of such a model take and return a 32-bit stream)
    stream_dtype: str = "engine"
    # logits <- logit_softcap * tanh(logits / logit_softcap) when set
    logit_softcap: float | None = None
    # a per-layer token input table that blocks read through the step's context (`ctx.token_side`)
    token_side: TokenSideSpec | None = None
    # (tensor name, rows): a table [rows, hidden] of vectors that schedule entries add to the stream
    # (`ScheduleEntry.add_vector`); needs stream_dtype="float32"
    pass_vectors: tuple[str, int] | None = None
    # tensor name of a matrix [hidden, 2 hidden] that maps [stream | embedding output] to the new stream before the
    # schedule entries that say `project_input`; needs stream_dtype="float32"
    pass_projection: str | None = None

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        if not self.schedule:
            raise ValueError("the schedule names no layer")
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, the model has {len(self.layers)}")
            if e.add_vector is not None and (self.pass_vectors is None or not 0 <= e.add_vector < self.pass_vectors[1]):
                raise ValueError(f"schedule entry {i}: add_vector={e.add_vector} names no row of the pass vectors")
            if e.project_input and self.pass_projection is None:
                raise ValueError(f"schedule entry {i}: project_input without a pass projection")
            if (e.add_input or e.add_vector is not None or e.project_input) and self.stream_dtype != "float32":
                raise ValueError(f"schedule entry {i}: additions to the stream need stream_dtype='float32'")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < i:
                    raise ValueError(f"schedule entry {i}: cache_of={e.cache_of} must name an earlier entry")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {i}: entry {e.cache_of} has no cache of its own")
