"""Small Finosun configurations for the tests, and model folders and runners made from them."""

from __future__ import annotations

import copy

import torch

import plain_finosun as pf
from conftest import device
from ludalix_helpers import replay, write_model  # noqa: F401  (step plans replayed through the step function)


def attention(heads, kv_heads, dim, vdim, scale, size, rot_dims=None, base=10000.0):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if size is not None:
        m["mask"] = dict(size=size)
    if rot_dims:
        m["rot"] = dict(dims=rot_dims, base=base)
    return m


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, base=10000.0):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale)
    if rot_dim:
        m["rot"] = dict(dims=rot_dim, base=base)
    return m


def moe(experts, identity, top, ff, limit, shared=None):
    """`shared`: (ff, limit) or None."""
    return dict(kind="moe", expert=dict(ff=ff, limit=limit), router=dict(experts=experts, identity=identity, top=top),
                shared=dict(ff=shared[0], limit=shared[1]) if shared else None)


def config(width, vocab, layers, loop=None, eps=2e-6):
    c = dict(architecture="Finosun", vocab=vocab, width=width, norm=dict(eps=eps),
             layers=[dict(type=t, mixer=m, mlp=f) for t, m, f in layers])
    if loop:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    return c


# A: a windowed layer in front of a loop of two layers that runs twice; values wider than keys; a part of each head
# rotated; two passing experts beside five real ones; a latent layer without feed-forward; one kv head for six
# heads with whole heads rotated and a routed layer without shared expert that takes a single expert
CFG_A = config(72, 211, [
    ("attention", attention(4, 2, 24, 40, 0.2, 9, rot_dims=8, base=900.0), moe(5, 2, 3, 48, 1.2, shared=(40, 2.5))),
    ("latent_attention", latent(3, 20, 12, 28, 40, 0.18, base=300.0), None),
    ("attention", attention(6, 1, 16, 16, 0.25, 13, rot_dims=16, base=50.0), moe(4, 0, 1, 32, 0.8)),
], loop=(1, 3, 2))
# B: the whole model is the loop (three passes; the first pass projects [embedding | embedding]); a window of 5
# under pages of 4; every router output chosen (top = experts + passing ones); a latent whose key row is no multiple
# of 8
CFG_B = config(64, 97, [
    ("attention", attention(6, 3, 16, 8, 0.3, 5, rot_dims=4, base=20.0), moe(2, 1, 3, 24, 2.0, shared=(16, 1.0))),
    ("latent_attention", latent(2, 8, 6, 8, 14, 0.2, base=100.0), moe(3, 3, 2, 40, 1.5, shared=(24, 3.0))),
], loop=(0, 2, 3), eps=1e-5)
# C: no loop; sizes that are no multiple of 8; a window of one page; a window of 3; values narrower than keys
CFG_C = config(100, 130, [
    ("latent_attention", latent(4, 36, 10, 20, 50, 0.1), moe(6, 1, 2, 36, 1.0, shared=(52, 2.0))),
    ("attention", attention(2, 2, 68, 20, 0.06, 16, rot_dims=34), moe(3, 0, 2, 44, 3.0, shared=(20, 0.5))),
    ("attention", attention(4, 1, 12, 12, 0.3, 3, rot_dims=12, base=7.0), None),
])
# D: values the other three make equal or leave out: a loop of one pass over one layer, one head, a window of one,
# attention without rotation and without a window, a latent without a rotated part, one expert, only passing
# experts beside it, heads of an odd size
CFG_D = config(48, 61, [
    ("attention", attention(1, 1, 32, 32, 0.2, 1, rot_dims=2), moe(1, 0, 1, 32, 1.0)),
    ("latent_attention", latent(1, 24, 0, 16, 24, 0.2), None),
    ("attention", attention(3, 3, 16, 24, 0.25, None), moe(1, 3, 2, 24, 1.1, shared=(8, 1.0))),
    ("latent_attention", latent(2, 8, 8, 8, 8, 0.3, base=3.0), moe(2, 0, 2, 16, 0.9)),
    ("attention", attention(2, 1, 15, 9, 0.25, 6, rot_dims=6, base=11.0), None),
], loop=(2, 3, 1))
# E: sizes the tensor-core attention kernels of the 16-bit path take: grouped heads of 64 and 128 with windows
# longer than a key tile, heads of 32 with values of 48, a latent whose key row (112 + 16) is a multiple of 16 and
# one whose row (56 + 8) is one while its rank is not a multiple of 16
CFG_E = config(96, 150, [
    ("attention", attention(4, 2, 64, 64, 0.125, 70, rot_dims=32), moe(4, 1, 2, 64, 1.5, shared=(48, 2.0))),
    ("attention", attention(4, 1, 128, 128, 0.09, 40, rot_dims=64, base=500.0), None),
    ("latent_attention", latent(4, 32, 16, 24, 112, 0.15), moe(8, 2, 4, 32, 1.5, shared=(64, 2.0))),
    ("attention", attention(2, 2, 32, 48, 0.2, 33, rot_dims=8), None),
    ("latent_attention", latent(2, 16, 8, 40, 56, 0.2, base=500.0), None),
], loop=(1, 4, 2))

CONFIGS = {"A": (CFG_A, 8), "B": (CFG_B, 4), "C": (CFG_C, 16), "D": (CFG_D, 8), "E": (CFG_E, 16)}  # config, page size


def cast(w, dtype):
    return w if dtype == "float32" else {n: t.to(getattr(torch, dtype)) for n, t in w.items()}


def weights_for(tag: str, dtype: str, seed: int = 0):
    cfg, page = CONFIGS[tag]
    w = pf.random_weights(cfg, seed=seed + sum(map(ord, tag)))
    return copy.deepcopy(cfg), cast(w, dtype), page


def every_output_chosen(cfg):
    """The configuration with every router output chosen (top = experts + passing ones).  The weights are the same;
    what falls away is the one discontinuity of the design: with a real choice, 16-bit rounding sends a token whose
    last chosen and first rejected outputs are nearly tied to another expert, and through the keys and values it
    then caches the difference reaches every later token.  Whole models in 16-bit are compared in this form; the
    choice itself is compared in 32-bit (whole models) and in 16-bit on the feed-forward alone, close calls left
    out."""
    c = copy.deepcopy(cfg)
    for L in c["layers"]:
        if L["mlp"] is not None:
            L["mlp"]["router"]["top"] = L["mlp"]["router"]["experts"] + L["mlp"]["router"].get("identity", 0)
    return c


def model_for(tag: str, dtype: str):
    """(config, weights, page size) of a whole-model comparison: as configured in 32-bit, with every router output
    chosen in 16-bit."""
    cfg, w, page = weights_for(tag, dtype)
    return (cfg if dtype == "float32" else every_output_chosen(cfg)), w, page


def make_runner(tmp_path, cfg, w, page, dtype, num_pages=64, max_requests=4, name="m", **kw):
    from ullm_b200.engine import ModelRunner

    d = write_model(str(tmp_path / f"{name}_{dtype}"), cfg, w)
    return ModelRunner(d, dtype=dtype, device=device(), page_size=page, num_pages=num_pages, max_requests=max_requests,
                       max_context=num_pages * page, max_step_tokens=64, poison_cache=True, **kw)


def oracle(ids, w, cfg) -> torch.Tensor:
    """Logits at every position, 64-bit arithmetic on the weights as given (rounded ones stay rounded)."""
    return pf.forward(cfg, {n: t.double() for n, t in w.items()}, ids).float()
