"""Small Pidenex configurations for the tests, and model folders and runners made from them."""

from __future__ import annotations

import copy

import torch

import plain_pidenex as pp
from conftest import device
from ludalix_helpers import replay, write_model  # noqa: F401  (step plans replayed through the step function)


def mask(size=None, pool=None):
    if size is None:
        return None
    m = dict(size=size)
    if pool:
        m["pool"] = pool
    return m


def _with_mask(m, size, pool=None):
    if size is not None:
        m["mask"] = mask(size, pool)
    return m


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, size, rot_dims=None, base=10000.0):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=scale)
    if rot_dim:
        m["rot"] = dict(dims=rot_dim if rot_dims is None else rot_dims, base=base)
    return _with_mask(m, size)


def attention(heads, kv_heads, dim, scale, size, pool=None):
    return _with_mask(dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale), size, pool)


def parallel(heads, kv_heads, dim, scale, size, width, left_scale=0.7, right_scale=1.3):
    left = _with_mask(dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale), size)
    return dict(left=left, right=dict(width=width), left_scale=left_scale, right_scale=right_scale)


def dense(ff):
    return dict(kind="dense", ff=ff)


def config(width, vocab, layers, loop=None, scale=5.0, eps=2e-6):
    c = dict(architecture="Pidenex", vocab=vocab, width=width, embedding=dict(scale=scale), norm=dict(eps=eps),
             layers=[dict(type=t, mixer=m, mlp=f) for t, m, f in layers])
    if loop:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    return c


# A: all three mixers; the last two run twice (a pass vector each, the embedding added again before the second);
# windows of 9, 13 and 11 over pages of 8; blocks of 4 pooled behind the last; rotation over a part of the rotated
# dimensions; a latent layer without feed-forward
CFG_A = config(72, 211, [
    ("parallel", parallel(4, 2, 24, 0.2, 9, 40), dense(96)),
    ("latent_attention", latent(3, 20, 12, 28, 40, 24, 0.18, 13, rot_dims=8, base=900.0), None),
    ("attention", attention(4, 2, 16, 0.25, 11, pool=4), dense(64)),
], loop=(1, 3, 2))
# B: the whole model is the loop (three passes, the first layer gets the first pass vector); one kv head for six
# heads; blocks of 3 under pages of 4 and a window of 5 (a block straddles pages; the window is shorter than two
# blocks); windows longer than most prompts; a parallel layer without feed-forward
CFG_B = config(64, 97, [
    ("attention", attention(6, 1, 16, 0.3, 5, pool=3), dense(48)),
    ("parallel", parallel(2, 2, 40, 0.15, 40, 24, 1.2, 0.4), None),
    ("latent_attention", latent(2, 8, 16, 8, 16, 32, 0.2, 40, base=300.0), dense(40)),
], loop=(0, 3, 3), eps=1e-5)
# C: no loop; sizes that are no multiple of 8; a window of one page with blocks of one page; a window of 3; a
# recurrence as wide as the model
CFG_C = config(100, 130, [
    ("latent_attention", latent(4, 36, 10, 20, 50, 30, 0.1, 16), dense(36)),
    ("attention", attention(2, 2, 68, 0.06, 16, pool=16), dense(52)),
    ("parallel", parallel(4, 1, 12, 0.3, 3, 100, 0.5, 0.9), dense(44)),
])
# D: values the other three make equal or leave out: a loop of one pass over one layer, one head, blocks of one
# token, a window of one, attention without a pool and without a window, a latent layer without a rotated part
CFG_D = config(48, 61, [
    ("attention", attention(1, 1, 32, 0.2, 1, pool=1), dense(32)),
    ("latent_attention", latent(1, 24, 0, 16, 24, 8, 0.2, None), None),
    ("attention", attention(3, 3, 16, 0.25, 6), None),
    ("parallel", parallel(1, 1, 16, 0.25, None, 8, 1.0, 1.0), dense(24)),
    ("attention", attention(2, 1, 24, 0.2, 7, pool=2), dense(40)),
], loop=(2, 3, 1))

CONFIGS = {"A": (CFG_A, 8), "B": (CFG_B, 4), "C": (CFG_C, 16), "D": (CFG_D, 8)}  # config, page size


def weights_for(tag: str, dtype: str, seed: int = 0):
    cfg, page = CONFIGS[tag]
    w = pp.random_weights(cfg, seed=seed + sum(map(ord, tag)))
    if dtype != "float32":
        w = {n: t.to(getattr(torch, dtype)) for n, t in w.items()}
    return copy.deepcopy(cfg), w, page


def cast(w, dtype):
    return w if dtype == "float32" else {n: t.to(getattr(torch, dtype)) for n, t in w.items()}


def make_runner(tmp_path, cfg, w, page, dtype, num_pages=64, max_requests=4, name="m", **kw):
    from ullm_b200.engine import ModelRunner

    d = write_model(str(tmp_path / f"{name}_{dtype}"), cfg, w)
    return ModelRunner(d, dtype=dtype, device=device(), page_size=page, num_pages=num_pages, max_requests=max_requests,
                       max_context=num_pages * page, max_step_tokens=64, poison_cache=True, **kw)


def oracle(ids, w, cfg) -> torch.Tensor:
    """Logits at every position, 64-bit arithmetic on the weights as given (rounded ones stay rounded)."""
    return pp.forward(cfg, {n: t.double() for n, t in w.items()}, ids).float()


# E: sizes the tensor-core attention kernel of the 16-bit path takes (rows of 16-byte multiples): grouped heads of
# 64 and 128 with windows longer than a key tile, blocks of 8 behind one of them, a latent whose key row (56 + 16)
# is no multiple of 16 while its rank is, values wider than one pass of the kernel (160 > 128)
CFG_E = config(96, 150, [
    ("parallel", parallel(4, 2, 64, 0.125, 70, 48, 0.8, 0.9), dense(72)),
    ("attention", attention(4, 1, 128, 0.09, 40, pool=8), None),
    ("latent_attention", latent(4, 32, 16, 24, 56, 48, 0.15, 90), dense(64)),
    ("latent_attention", latent(2, 16, 16, 40, 160, 32, 0.2, 33, base=500.0), None),
], loop=(1, 3, 2))
CONFIGS["E"] = (CFG_E, 16)
