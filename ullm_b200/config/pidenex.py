"""Typed configuration of the Pidenex decoder, read from the keys of its config.json, and its translation into a
ModelSpec.

The design: a scaled token embedding; a list of layers, each x <- x + norm_1b(mixer(norm_1(x))) and, if it has a
feed-forward, x <- x + norm_2b(ff(norm_2(x))), with layer norms (a weight, no bias) on a 32-bit residual stream.
A range of layers may run several times in a row with the same weights (`loop`), every pass with caches and state
of its own; before every pass but the first the embedding's output is added to the stream again, and before every
pass a vector of that pass (`loop.step`).  Mixers:

* `latent_attention`: queries and keys / values through low-rank latents, one rotated key part shared by the
  heads, interleaved rotation, a sliding window;
* `attention`: grouped heads whose values are their keys, no positions, a sliding window plus one mean key / value
  per block of `mask.pool` tokens that lies wholly before the window;
* `parallel`: `left` (grouped heads, values = keys before their norm, q and k normed over the whole projection, a
  distance bias with a slope per head, a sliding window, a sigmoid output gate) beside `right` (a minGRU with
  per-request state), summed with a scale each.

Feed-forward: `dense`, down(act(up(x))) with the two-number activation of `mlp.act`.  A final layer norm and an
output head.

config.json keys: architecture, vocab, width, embedding.scale, norm.eps, loop{start, stop, times} (optional),
layers[] with type, mixer{...}, mlp{kind, ff} | null.  Tensor names: embed, loop.step, l<i>.norm1, norm1b, norm2,
norm2b, l<i>.mix.*, l<i>.mlp.*, final.norm, head.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .specs import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry

ARCHITECTURE = "Pidenex"
# constant the design fixes: head h of H loses 2^(-SLOPE_EXPONENT (h + 1) / H) per position of distance
SLOPE_EXPONENT = 8.0
MIXER_TYPES = ("latent_attention", "attention", "parallel")


class PidenexConfigError(ValueError):
    pass


def _need(d, key: str, where: str, kind=(int, float)):
    if not isinstance(d, dict) or key not in d:
        raise PidenexConfigError(f"config.json: {where} lacks {key!r}")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, kind):
        raise PidenexConfigError(f"config.json: {where}.{key} = {v!r} is not a number")
    return v


def _positive_int(d, key: str, where: str) -> int:
    v = _need(d, key, where, (int,))
    if v <= 0:
        raise PidenexConfigError(f"config.json: {where}.{key} must be positive, got {v}")
    return v


def _mask(mix: dict, where: str, pool_allowed: bool) -> tuple[int | None, int]:
    """(window or None, pool or 0) of a mixer's `mask`."""
    mask = mix.get("mask")
    if mask is None:
        return None, 0
    if not isinstance(mask, dict):
        raise PidenexConfigError(f"config.json: {where}.mask must be an object")
    size = _positive_int(mask, "size", where + ".mask")
    pool = 0
    if mask.get("pool") is not None:
        if not pool_allowed:
            raise PidenexConfigError(f"config.json: {where}.mask.pool: this mixer's scores depend on the distance, "
                                     f"which a pooled block does not have")
        pool = _positive_int(mask, "pool", where + ".mask")
    return size, pool


def _check_grouped(m: dict, where: str) -> None:
    for k in ("heads", "kv_heads", "dim", "vdim"):
        _positive_int(m, k, where)
    if m["heads"] % m["kv_heads"]:
        raise PidenexConfigError(f"config.json: {where}.heads is no multiple of kv_heads")
    if m["vdim"] != m["dim"]:
        raise PidenexConfigError(f"config.json: {where}: the values are the keys, so vdim must equal dim")
    _need(m, "scale", where)


@dataclass(frozen=True)
class PidenexLayer:
    type: str
    mixer: dict[str, Any]
    mlp: dict[str, Any] | None


@dataclass(frozen=True)
class PidenexConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: tuple[PidenexLayer, ...]
    loop: tuple[int, int, int] | None  # (start, stop, times)
    dtype: str = "bfloat16"
    max_positions: int = 1 << 30  # positions are computed, not tabulated: the context is the engine's choice
    raw: dict[str, Any] = field(default_factory=dict, hash=False, compare=False)

    @staticmethod
    def from_dict(d: dict[str, Any]) -> "PidenexConfig":
        vocab, width = _positive_int(d, "vocab", "the config"), _positive_int(d, "width", "the config")
        scale = float(_need(d.get("embedding"), "scale", "embedding"))
        eps = float(_need(d.get("norm"), "eps", "norm"))
        if eps <= 0:
            raise PidenexConfigError("config.json: norm.eps must be positive")
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise PidenexConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]"
            if not isinstance(L, dict) or L.get("type") not in MIXER_TYPES:
                raise PidenexConfigError(f"config.json: {where}.type must be one of {MIXER_TYPES}")
            mix = L.get("mixer")
            if not isinstance(mix, dict):
                raise PidenexConfigError(f"config.json: {where} lacks 'mixer'")
            mw = where + ".mixer"
            if L["type"] == "latent_attention":
                for k in ("heads", "dim", "vdim", "kv_rank", "q_rank"):
                    _positive_int(mix, k, mw)
                rot = _need(mix, "rot_dim", mw, (int,))
                if rot < 0:
                    raise PidenexConfigError(f"config.json: {mw}.rot_dim must not be negative")
                _need(mix, "scale", mw)
                if rot:
                    dims = _positive_int(mix.get("rot"), "dims", mw + ".rot")
                    if dims % 2 or dims > rot:
                        raise PidenexConfigError(f"config.json: {mw}.rot.dims must be even and at most rot_dim")
                    if float(_need(mix.get("rot"), "base", mw + ".rot")) <= 0:
                        raise PidenexConfigError(f"config.json: {mw}.rot.base must be positive")
                _mask(mix, mw, True)
            elif L["type"] == "attention":
                _check_grouped(mix, mw)
                _mask(mix, mw, True)
            else:
                left, right = mix.get("left"), mix.get("right")
                if not isinstance(left, dict) or not isinstance(right, dict):
                    raise PidenexConfigError(f"config.json: {mw} lacks 'left' or 'right'")
                _check_grouped(left, mw + ".left")
                _mask(left, mw + ".left", False)
                _positive_int(right, "width", mw + ".right")
                _need(mix, "left_scale", mw)
                _need(mix, "right_scale", mw)
            mlp = L.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise PidenexConfigError(f"config.json: {where}.mlp.kind must be 'dense'")
                _positive_int(mlp, "ff", where + ".mlp")
            layers.append(PidenexLayer(L["type"], dict(mix), dict(mlp) if mlp is not None else None))
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            a, b = _need(lp, "start", "loop", (int,)), _need(lp, "stop", "loop", (int,))
            times = _positive_int(lp, "times", "loop")
            if not 0 <= a < b <= len(layers):
                raise PidenexConfigError(f"config.json: loop covers layers {a} .. {b - 1}, the model has {len(layers)}")
            loop = (a, b, times)
        dt = str(d.get("dtype", d.get("torch_dtype", "bfloat16"))).replace("torch.", "")
        if dt not in ("bfloat16", "float32", "float16"):
            raise PidenexConfigError(f"Unsupported dtype {dt!r}")
        return PidenexConfig(vocab, width, scale, eps, tuple(layers), loop, dt, raw=dict(d))

    def to_dict(self) -> dict[str, Any]:
        return dict(self.raw)


def _grouped_attention(W: int, m: dict, eps: float, window, pool: int, left: bool) -> MixerSpec:
    names = dict(q="q", k="k", o="o", g="g", q_norm="q.norm", k_norm="k.norm")
    return MixerSpec("kv_shared_attention", dict(
        hidden_size=W, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], scale=float(m["scale"]),
        window=window, pool=pool, whole_norm=left, norm_eps=eps, slope_exponent=SLOPE_EXPONENT if left else None,
        gated=left, names=names))


def pidenex_model_spec(cfg: PidenexConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    bare = dict(param="")  # a norm's weight is named by its prefix alone

    def norm():
        return NormSpec("layernorm", W, eps, bare)

    layers = []
    for L in cfg.layers:
        mix = L.mixer
        if L.type == "latent_attention":
            window, pool = _mask(mix, "mixer", True)
            position = None
            if mix["rot_dim"]:
                position = PositionSpec("rope_computed", rotary_dim=int(mix["rot"]["dims"]), theta=float(mix["rot"]["base"]),
                                        args=dict(interleaved=True))
            mixer = MixerSpec("latent_attention", dict(
                hidden_size=W, num_heads=mix["heads"], head_dim=mix["dim"], rot_dim=mix["rot_dim"],
                value_dim=mix["vdim"], q_rank=mix["q_rank"], kv_rank=mix["kv_rank"], position=position,
                scale=float(mix["scale"]), window=window, pool=pool, norm_eps=eps,
                names=dict(dq="dq", dq_norm="dq.norm", uq="uq", dkv="dkv", dkv_norm="dkv.norm", uk="uk", uv="uv", o="o")))
        elif L.type == "attention":
            window, pool = _mask(mix, "mixer", True)
            mixer = _grouped_attention(W, mix, eps, window, pool, left=False)
        else:
            window, _pool = _mask(mix["left"], "mixer.left", False)
            mixer = MixerSpec("parallel_mixers", dict(
                hidden_size=W, left=_grouped_attention(W, mix["left"], eps, window, 0, left=True),
                right=MixerSpec("mingru", dict(hidden_size=W, width=mix["right"]["width"],
                                               names=dict(z="z", z_bias="z.b", x="x", x_bias="x.b", g="g", o="o"))),
                left_scale=float(mix["left_scale"]), right_scale=float(mix["right_scale"]),
                names=dict(left="left.", right="right.")))
        ff = None
        if L.mlp is not None:
            ff = FeedForwardSpec("dense_mlp", dict(hidden_size=W, intermediate_size=L.mlp["ff"], activation="xielu",
                                                   names=dict(up="up", down="down", act="act")))
        layers.append(LayerSpec(
            block="sandwich_residual", mixer=mixer, feed_forward=ff, mixer_norm=norm(),
            feed_forward_norm=norm() if ff is not None else None,
            names=dict(mixer="mix.", feed_forward="mlp.", mixer_norm="norm1", mixer_out_norm="norm1b",
                       feed_forward_norm="norm2", feed_forward_out_norm="norm2b"),
            block_args=dict(mixer_out_norm=norm(), feed_forward_out_norm=norm() if ff is not None else None)))
    n = len(layers)
    if cfg.loop is None:
        schedule = [ScheduleEntry(i) for i in range(n)]
        pass_vectors = None
    else:
        a, b, times = cfg.loop
        schedule = [ScheduleEntry(i) for i in range(a)]
        for t in range(times):
            # a pass starts: the embedding's output again (not before the first), then the pass's vector
            schedule += [ScheduleEntry(i, None, add_input=(i == a and t > 0), add_vector=t if i == a else None)
                         for i in range(a, b)]
        schedule += [ScheduleEntry(i) for i in range(b, n)]
        pass_vectors = ("loop.step", times)
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=W, vocab_size=cfg.vocab, layers=layers, schedule=schedule,
        final_norm=norm(), tie_embeddings=False, max_positions=cfg.max_positions, dtype=cfg.dtype,
        embedding_name="embed", layer_name="l{}.", final_norm_name="final.norm", head_name="head",
        embedding_param="", head_param="", embedding_scale=cfg.embedding_scale, stream_dtype="float32",
        pass_vectors=pass_vectors)
