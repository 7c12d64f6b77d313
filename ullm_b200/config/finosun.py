"""Typed configuration of the Finosun decoder, read from the keys of its config.json, and its translation into a
ModelSpec.

The design: a token embedding that is also the output head; a list of pre-norm layers on a 32-bit residual stream,
x <- x + s1 * mixer(norm1(x)) and, if the layer has a feed-forward, x <- x + s2 * ff(norm2(x)), with RMS norms and a
scale per channel (s1, s2) on each sub-layer's output.  A range of layers may run several times in a row with the
same weights (`loop`), every pass with caches of its own; right before the first layer of every pass the stream is
replaced by a projection of [stream | embedding output] (`loop.in`, [width, 2 width]).  Mixers:

* `attention`: grouped heads; q and k pass an RMS norm over the WHOLE projection (a weight per channel) before
  the first `rot.dims` dimensions of every head are rotated in neighbouring pairs (2i, 2i + 1); every head's value
  is divided by its root mean square (no weight) and cached so; scores times `scale` times a learned number per
  head; a sliding window.
* `latent_attention`: queries projected directly and laid out per head as [dim unrotated | rot_dim rotated]; keys
  and values from one RMS-normed latent of `kv_rank` per token plus ONE rotated key part shared by all heads
  (pairs (i, i + rot_dim / 2)); causal; the concatenated heads pass a sigmoid gate read from the mixer's input.

Feed-forward `moe`: `experts` routed experts (clamped gate and up, g * sigmoid(1.702 g) * (u + 1)), of which each
token takes `top`; the softmax over all router outputs gives the weights (not renormalized), the choice adds a
correction per output; the last `identity` router outputs stand for experts that pass their input; a shared expert
of the same form runs for every token, times a sigmoid gate of one number per token.  A final RMS norm.

config.json keys: architecture, vocab, width, norm.eps, loop{start, stop, times} (optional), layers[] with type,
mixer{...}, mlp{kind, expert{ff, limit}, router{experts, identity, top}, shared{ff, limit} | null} | null.
Tensor names: embed, loop.in, l<i>.norm1, norm2, ls1, ls2, l<i>.mix.*, l<i>.mlp.*, final.norm.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .specs import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry

ARCHITECTURE = "Finosun"
# constant the design fixes: the slope of the experts' gate, g * sigmoid(ACT_SLOPE * g)
ACT_SLOPE = 1.702
MIXER_TYPES = ("attention", "latent_attention")


class FinosunConfigError(ValueError):
    pass


def _need(d, key: str, where: str, kind=(int, float)):
    if not isinstance(d, dict) or key not in d:
        raise FinosunConfigError(f"config.json: {where} lacks {key!r}")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, kind):
        raise FinosunConfigError(f"config.json: {where}.{key} = {v!r} is not a number")
    return v


def _positive_int(d, key: str, where: str) -> int:
    v = _need(d, key, where, (int,))
    if v <= 0:
        raise FinosunConfigError(f"config.json: {where}.{key} must be positive, got {v}")
    return v


def _positive(d, key: str, where: str) -> float:
    v = float(_need(d, key, where))
    if not v > 0:
        raise FinosunConfigError(f"config.json: {where}.{key} must be positive, got {v}")
    return v


def _window(mix: dict, where: str) -> int | None:
    mask = mix.get("mask")
    if mask is None:
        return None
    if not isinstance(mask, dict):
        raise FinosunConfigError(f"config.json: {where}.mask must be an object")
    return _positive_int(mask, "size", where + ".mask")


def _rotation(mix: dict, where: str, most: int) -> tuple[int, float]:
    """(rotated dimensions, base) of a mixer's `rot`; (0, 0) when it has none."""
    rot = mix.get("rot")
    if rot is None:
        return 0, 0.0
    dims = _positive_int(rot, "dims", where + ".rot")
    if dims % 2 or dims > most:
        raise FinosunConfigError(f"config.json: {where}.rot.dims must be even and at most {most}")
    return dims, _positive(rot, "base", where + ".rot")


def _check_expert(e, where: str) -> None:
    _positive_int(e, "ff", where)
    _positive(e, "limit", where)


@dataclass(frozen=True)
class FinosunLayer:
    type: str
    mixer: dict[str, Any]
    mlp: dict[str, Any] | None


@dataclass(frozen=True)
class FinosunConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[FinosunLayer, ...]
    loop: tuple[int, int, int] | None  # (start, stop, times)
    dtype: str = "bfloat16"
    max_positions: int = 1 << 30  # positions are computed, not tabulated: the context is the engine's choice
    raw: dict[str, Any] = field(default_factory=dict, hash=False, compare=False)

    @staticmethod
    def from_dict(d: dict[str, Any]) -> "FinosunConfig":
        vocab, width = _positive_int(d, "vocab", "the config"), _positive_int(d, "width", "the config")
        eps = _positive(d.get("norm"), "eps", "norm")
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise FinosunConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]"
            if not isinstance(L, dict) or L.get("type") not in MIXER_TYPES:
                raise FinosunConfigError(f"config.json: {where}.type must be one of {MIXER_TYPES}")
            mix = L.get("mixer")
            if not isinstance(mix, dict):
                raise FinosunConfigError(f"config.json: {where} lacks 'mixer'")
            mw = where + ".mixer"
            if L["type"] == "attention":
                for k in ("heads", "kv_heads", "dim", "vdim"):
                    _positive_int(mix, k, mw)
                if mix["heads"] % mix["kv_heads"]:
                    raise FinosunConfigError(f"config.json: {mw}.heads is no multiple of kv_heads")
                _rotation(mix, mw, mix["dim"])
            else:
                for k in ("heads", "dim", "vdim", "kv_rank"):
                    _positive_int(mix, k, mw)
                rot = _need(mix, "rot_dim", mw, (int,))
                if rot < 0 or rot % 2:
                    raise FinosunConfigError(f"config.json: {mw}.rot_dim must be even and not negative")
                if rot:
                    dims, _ = _rotation(mix, mw, rot)
                    if dims != rot:
                        raise FinosunConfigError(f"config.json: {mw}.rot.dims must equal rot_dim (the whole shared "
                                                 f"part is rotated)")
            _need(mix, "scale", mw)
            _window(mix, mw)
            mlp = L.get("mlp")
            if mlp is not None:
                fw = where + ".mlp"
                if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
                    raise FinosunConfigError(f"config.json: {fw}.kind must be 'moe'")
                _check_expert(mlp.get("expert"), fw + ".expert")
                r = mlp.get("router")
                E, top = _positive_int(r, "experts", fw + ".router"), _positive_int(r, "top", fw + ".router")
                ident = r.get("identity", 0)
                if isinstance(ident, bool) or not isinstance(ident, int) or ident < 0:
                    raise FinosunConfigError(f"config.json: {fw}.router.identity must be a count")
                if top > E + ident:
                    raise FinosunConfigError(f"config.json: {fw}.router.top is more than there are router outputs")
                if mlp.get("shared") is not None:
                    _check_expert(mlp["shared"], fw + ".shared")
            layers.append(FinosunLayer(L["type"], dict(mix), dict(mlp) if mlp is not None else None))
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            a, b = _need(lp, "start", "loop", (int,)), _need(lp, "stop", "loop", (int,))
            times = _positive_int(lp, "times", "loop")
            if not 0 <= a < b <= len(layers):
                raise FinosunConfigError(f"config.json: loop covers layers {a} .. {b - 1}, the model has {len(layers)}")
            loop = (a, b, times)
        dt = str(d.get("dtype", d.get("torch_dtype", "bfloat16"))).replace("torch.", "")
        if dt not in ("bfloat16", "float32", "float16"):
            raise FinosunConfigError(f"Unsupported dtype {dt!r}")
        return FinosunConfig(vocab, width, eps, tuple(layers), loop, dt, raw=dict(d))

    def to_dict(self) -> dict[str, Any]:
        return dict(self.raw)


def _expert_ff(W: int, e: dict) -> FeedForwardSpec:
    return FeedForwardSpec("gated_mlp", dict(hidden_size=W, intermediate_size=e["ff"], activation="swiglu_clamped",
                                             limit=float(e["limit"]), alpha=ACT_SLOPE,
                                             names=dict(gate="gate", up="up", down="down")))


def finosun_model_spec(cfg: FinosunConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    bare = dict(param="")  # a norm's weight is named by its prefix alone

    def norm():
        return NormSpec("rmsnorm", W, eps, bare)

    layers = []
    for L in cfg.layers:
        mix = L.mixer
        window = _window(mix, "mixer")
        if L.type == "attention":
            dims, base = _rotation(mix, "mixer", mix["dim"])
            position = PositionSpec("rope_computed", rotary_dim=dims, theta=base,
                                    args=dict(interleaved=True)) if dims else None
            mixer = MixerSpec("paged_attention", dict(
                hidden_size=W, num_heads=mix["heads"], num_kv_heads=mix["kv_heads"], head_dim=mix["dim"],
                value_dim=mix["vdim"], qk_norm=NormSpec("rmsnorm", mix["dim"], eps, bare), whole_norm=True,
                value_unit_norm=True, head_temperature=True, position=position, window=window,
                scale=float(mix["scale"]), norm_eps=eps,
                names=dict(q="q", k="k", v="v", o="o", q_norm="q.norm", k_norm="k.norm", temp="temp")))
        else:
            r = mix["rot_dim"]
            position = PositionSpec("rope_computed", rotary_dim=r, theta=float(mix["rot"]["base"]),
                                    args=dict(interleaved=False)) if r else None
            mixer = MixerSpec("latent_attention", dict(
                hidden_size=W, num_heads=mix["heads"], head_dim=mix["dim"], rot_dim=r, value_dim=mix["vdim"],
                q_rank=None, kv_rank=mix["kv_rank"], position=position, scale=float(mix["scale"]), window=window,
                gated=True, norm_eps=eps,
                names=dict(q="q", dkv="dkv", dkv_norm="dkv.norm", uk="uk", uv="uv", g="g", o="o")))
        ff = None
        if L.mlp is not None:
            f = L.mlp
            shared = _expert_ff(W, f["shared"]) if f.get("shared") is not None else None
            ff = FeedForwardSpec("routed_experts", dict(
                hidden_size=W, intermediate_size=f["expert"]["ff"], num_experts=f["router"]["experts"],
                top=f["router"]["top"], activation="swiglu_clamped", limit=float(f["expert"]["limit"]), alpha=ACT_SLOPE,
                scores="softmax", renormalize=False, weight_on="output", correction=True,
                identity=int(f["router"].get("identity", 0)), shared=shared, shared_gate=shared is not None,
                names=dict(router="router", correction="correction", gate="e{}.gate", up="e{}.up", down="e{}.down",
                           shared="shared.", shared_gate="shared.sg")))
        layers.append(LayerSpec(
            block="prenorm_scaled", mixer=mixer, feed_forward=ff, mixer_norm=norm(),
            feed_forward_norm=norm() if ff is not None else None,
            names=dict(mixer="mix.", feed_forward="mlp.", mixer_norm="norm1", feed_forward_norm="norm2",
                       mixer_scale="ls1", feed_forward_scale="ls2"),
            block_args=dict(layer_scale=True)))
    n = len(layers)
    if cfg.loop is None:
        schedule = [ScheduleEntry(i) for i in range(n)]
        pass_projection = None
    else:
        a, b, times = cfg.loop
        schedule = [ScheduleEntry(i) for i in range(a)]
        for _t in range(times):
            # a pass starts: the stream becomes a projection of [stream | embedding output]
            schedule += [ScheduleEntry(i, None, project_input=(i == a)) for i in range(a, b)]
        schedule += [ScheduleEntry(i) for i in range(b, n)]
        pass_projection = "loop.in"
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=W, vocab_size=cfg.vocab, layers=layers, schedule=schedule,
        final_norm=norm(), tie_embeddings=True, max_positions=cfg.max_positions, dtype=cfg.dtype,
        embedding_name="embed", layer_name="l{}.", final_norm_name="final.norm", head_name="head",
        embedding_param="", head_param="", stream_dtype="float32", pass_projection=pass_projection)
