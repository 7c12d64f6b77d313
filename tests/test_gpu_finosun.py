"""The Finosun decoder in the engine against the plain implementation (tests/plain_finosun.py): each mechanism
alone, whole prompts against token-by-token decoding and portions down to two tokens, unequal batches with pages
and request slots that are used again, the edges of windows (with weights made so that one key decides), a far key
among hundreds, the first tokens, long decoding, and greedy generation through the entry point and the scheduler."""

import copy

import pytest
import torch

import plain_finosun as pf
from conftest import device
from finosun_helpers import (CONFIGS, attention, cast, config, every_output_chosen, latent, make_runner, model_for, moe,
                             oracle, replay, weights_for, write_model)
from helpers import TOL, TOL_RMS, assert_close, errors, random_ids
from ludalix_helpers import assert_rows_close

pytestmark = pytest.mark.gpu


def close(got, ref, dtype, what):
    """A part alone: 32-bit to 3e-5 of the largest value; bfloat16 within the limits the whole models get."""
    if dtype != "float32":
        return assert_close(got, ref, dtype, what)
    mx, _ = errors(got, ref)
    assert torch.isfinite(got.float()).all(), f"{what}: non-finite"
    assert mx <= 3e-5, f"{what}: max err {mx:.2e} of scale"


def rand(shape, seed, dtype, scale=1.0):
    t = torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale
    return t.to(getattr(torch, dtype)).to(device())


def first_run_of(cfg, layer):
    return [i for i, _ in pf.layer_runs(cfg)].index(layer)


def mixer_in_steps(r, cfg, layer, x, cuts):
    """The mixer of `layer` (through the cache of its first run) on the rows x, cut into steps at `cuts`."""
    from ullm_b200.engine import StepEntry

    run = first_run_of(cfg, layer)
    got = []
    r.add_request("a")
    for a, b in zip((0,) + tuple(cuts), tuple(cuts) + (x.shape[0],)):
        e = [StepEntry("a", [0] * (b - a), [])]
        ctx = r.prepare(e)
        caches = r.cache.layer_caches(ctx.groups)
        got.append(r.model.blocks[layer].mixer.forward(x[a:b].clone(), ctx, caches[run]).float().cpu().clone())
        r.commit(e)
    r.check_device_status()
    r.end_request("a")
    return torch.cat(got)


# ---------------------------------------------------------------------------------------------------------
# each mechanism alone
# ---------------------------------------------------------------------------------------------------------
MIXERS = [(tag, i) for tag, (cfg, _) in CONFIGS.items() for i in range(len(cfg["layers"]))]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag,layer", MIXERS)
def test_every_mixer_alone(tmp_path, dtype, tag, layer):
    """Random rows in four steps (29, 2, 1 and 15 tokens: windows of 1 to 40 pass their edges inside a portion and
    between portions) against the mixer run whole."""
    cfg, w, page = weights_for(tag, dtype)
    r = make_runner(tmp_path, cfg, w, page, dtype)
    x = rand((47, cfg["width"]), 5 + layer, dtype)
    wd = {n: t.double() for n, t in w.items()}
    L = cfg["layers"][layer]
    ref = pf.mixer(L["type"], x.double().cpu(), L["mixer"], wd, f"l{layer}.mix.", cfg["norm"]["eps"]).float()
    got = mixer_in_steps(r, cfg, layer, x, (29, 31, 32))
    close(got, ref, dtype, f"{tag} layer {layer} ({L['type']})")


def _ctx_for(r):
    from ullm_b200.engine.batch import Workspace

    class Ctx:
        workspace = Workspace(r.device, max_tokens=32, max_requests=4)

    return Ctx()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "B", "C", "D", "E"])
def test_every_feed_forward_alone(tmp_path, dtype, tag):
    """Router, correction, passing experts, clamped experts, the gated shared expert.  Rows whose choice is a close
    call in the plain model do not count in 16-bit."""
    cfg, w, page = weights_for(tag, dtype)
    r = make_runner(tmp_path, cfg, w, page, dtype)
    x = rand((21, cfg["width"]), 8, dtype, 1.5)
    wd = {k: t.double() for k, t in w.items()}
    for l, L in enumerate(cfg["layers"]):
        if L["mlp"] is None:
            continue
        pre, f = f"l{l}.mlp.", L["mlp"]
        ref = pf.routed_ff(x.double().cpu(), f, wd, pre).float()
        got = r.model.blocks[l].feed_forward.forward(x.clone(), _ctx_for(r)).float().cpu()
        s = (torch.softmax(x.double().cpu() @ wd[pre + "router"].T, -1) + wd[pre + "correction"]).sort(-1, descending=True).values
        top = f["router"]["top"]
        clear = torch.ones(21, dtype=torch.bool) if top == s.shape[1] else (s[:, top - 1] - s[:, top]) > (
            0.0 if dtype == "float32" else 0.002)
        assert clear.sum() >= 8
        close(got[clear], ref[clear], dtype, f"{tag} layer {l} feed-forward")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "C", "E"])
def test_a_feed_forward_adds_itself_to_the_stream_as_the_separate_kernels_do(tmp_path, dtype, tag):
    """The routed feed-forward's last kernel in its form that adds to the 32-bit stream with a scale per channel and
    leaves the next norm's rows, against the plain feed-forward, the sum and the norm in 64-bit; the rows of the
    next norm may overwrite the feed-forward's own input."""
    cfg, w, page = weights_for(tag, dtype)
    cfg = cfg if dtype == "float32" else every_output_chosen(cfg)
    r = make_runner(tmp_path, cfg, w, page, dtype)
    W = cfg["width"]
    x = rand((19, W), 8, dtype, 1.5)
    wd = {k: t.double() for k, t in w.items()}
    g = torch.Generator().manual_seed(4)
    stream0 = torch.randn(19, W, generator=g)
    scale = 0.5 + torch.rand(W, generator=g)
    w2 = 1.0 + 0.2 * torch.randn(W, generator=g)
    for l, L in enumerate(cfg["layers"]):
        if L["mlp"] is None:
            continue
        ref = stream0.double() + scale.double() * pf.routed_ff(x.double().cpu(), L["mlp"], wd, f"l{l}.mlp.")
        ref_norm = pf.rms_norm(ref, w2.double(), 3e-6)
        stream = stream0.clone().to(device())
        rows = x.clone()  # (the next norm's rows take the input's place)
        ok = r.model.blocks[l].feed_forward.forward_add(rows, _ctx_for(r), stream, scale.to(device()),
                                                        (w2.to(device()), 3e-6, rows))
        assert ok
        close(stream, ref.float(), dtype, f"{tag} layer {l}: stream")
        close(rows, ref_norm.float(), dtype, f"{tag} layer {l}: next norm")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_large_correction_decides_the_choice_but_not_the_weight(tmp_path, dtype):
    """One router output gets a correction far above every score: every token takes it, with its own small score as
    the weight; once it is a real expert, once a passing one."""
    for ident, favoured in ((1, 1), (2, 4)):
        cfg = config(40, 50, [("attention", attention(2, 1, 16, 16, 0.25, 4), moe(3, ident, 1, 24, 1.0, shared=(16, 1.0)))])
        w = pf.random_weights(cfg, seed=12 + ident)
        w["l0.mlp.correction"] = torch.zeros(3 + ident)
        w["l0.mlp.correction"][favoured] = 5.0
        w["l0.mlp.router"][favoured] = -w["l0.mlp.router"][0]  # (often the smallest score)
        w = cast(w, dtype)
        r = make_runner(tmp_path, cfg, w, 8, dtype, name=f"c{ident}")
        x = rand((9, 40), 3, dtype, 2.0)
        wd = {k: t.double() for k, t in w.items()}
        chosen, weight = pf.route(x.double().cpu(), wd, "l0.mlp.", 1)
        assert (chosen == favoured).all() and float(weight.min()) < 0.05  # (chosen also where its score is tiny)
        ref = pf.routed_ff(x.double().cpu(), cfg["layers"][0]["mlp"], wd, "l0.mlp.").float()
        close(r.model.blocks[0].feed_forward.forward(x.clone(), _ctx_for(r)), ref, dtype, f"correction on output {favoured}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_head_factors_value_norm_and_layer_scale_each_show(tmp_path, dtype):
    """A model whose head factors, layer scales and values are far from what leaves them unseen (factors 0.2 to 3,
    scales 0.1 to 2, values a hundred times too large for a model that did not divide them by their root mean
    square): whole prompt against the plain model, and the plain model itself changes when one is left out."""
    cfg = config(56, 80, [("attention", attention(4, 2, 16, 24, 0.25, 7, rot_dims=6, base=40.0), moe(3, 1, 2, 24, 1.0, shared=(16, 1.5))),
                          ("latent_attention", latent(2, 12, 4, 10, 20, 0.2, base=30.0), None)], loop=(0, 2, 2))
    w = pf.random_weights(cfg, seed=33)
    w["l0.mix.temp"] = torch.tensor([0.2, 3.0, 1.0, 0.5])
    w["l0.mix.v"] = w["l0.mix.v"] * 100.0
    for n in ("l0.ls1", "l0.ls2", "l1.ls1"):
        w[n] = torch.linspace(0.1, 2.0, 56)
    w = cast(w, dtype)
    cfg = cfg if dtype == "float32" else every_output_chosen(cfg)
    ids = random_ids(80, 40, 2)
    ref = oracle(ids, w, cfg)
    for name, val in (("l0.mix.temp", torch.ones(4)), ("l0.ls2", torch.ones(56)), ("l1.ls1", torch.ones(56))):
        other = dict(w)
        other[name] = val.to(w[name].dtype)
        assert (oracle(ids, other, cfg) - ref).abs().max() > 5 * TOL[dtype] * ref.abs().max(), name
    r = make_runner(tmp_path, cfg, w, 8, dtype)
    got = replay(r, {"a": ids}, [[("a", 17)], [("a", 2)], [("a", 21)]])["a"]
    assert_rows_close(got, ref, dtype, "factors, scales and value norm")


# ---------------------------------------------------------------------------------------------------------
# whole prompts, token-by-token decoding, portions
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "B", "C", "D", "E"])
def test_whole_decode_and_portions_agree_with_the_plain_model(tmp_path, dtype, tag):
    cfg, w, page = model_for(tag, dtype)
    r = make_runner(tmp_path, cfg, w, page, dtype, num_pages=96 if tag == "B" else 64)
    n = 75 if tag != "E" else 150  # (E: the window of 70 must pass over prompt and decoded tokens)
    ids = random_ids(cfg["vocab"], n, 11)
    ref = oracle(ids, w, cfg)
    plans = {
        "whole": [[("a", n)]],
        "decode": [[("b", 3)]] + [[("b", 1)] for _ in range(n - 3)],
        "portions": [[("c", k)] for k in (2, 2, 3, 7, 2, 16, 1, 1, 2, 31, 8) + ((70, 5) if n == 150 else ())],
        "one by one": [[("d", 1)] for _ in range(n)],
    }
    assert sum(k for (_, k), in plans["portions"]) == n
    for name, plan in plans.items():
        rid = plan[0][0][0]
        got = replay(r, {rid: ids}, plan)[rid]
        assert_rows_close(got, ref, dtype, f"{tag} {name}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "E"])
def test_unequal_batches_with_pages_and_slots_used_again(tmp_path, dtype, tag):
    """Three request slots and a pool that cannot hold all requests at once: six requests of unequal length come
    and go, portions of some beside single tokens of others; every request equals itself run alone."""
    cfg, w, page = model_for(tag, dtype)
    pages = 24 if tag == "A" else 17
    r = make_runner(tmp_path, cfg, w, page, dtype, num_pages=pages, max_requests=3)
    lens = dict(a=50, b=9, c=61, d=2, e=33, f=17)
    reqs = {k: random_ids(cfg["vocab"], n, 40 + n) for k, n in lens.items()}
    plan = [
        [("a", 20), ("b", 2)],
        [("a", 1), ("b", 5), ("c", 30)],
        [("b", 2), ("a", 9), ("c", 1)],          # b ends: its slot and pages go back
        [("d", 2), ("c", 1), ("a", 1)],          # d takes them, and ends at once
        [("e", 16), ("a", 19)],                  # a ends
        [("c", 29), ("e", 1), ("f", 2)],         # c ends; f starts on a slot and pages that were used
        [("f", 15), ("e", 16)],
    ]
    got = replay(r, reqs, plan)
    for k in reqs:
        assert_rows_close(got[k], oracle(reqs[k], w, cfg), dtype, f"request {k}")
    assert not r.cache.requests
    assert all(r.cache.num_free_pages(g) == n for g, n in enumerate(r.cache.group_pages))


# ---------------------------------------------------------------------------------------------------------
# edges: windows, page borders; weights made so that one key decides
# ---------------------------------------------------------------------------------------------------------
def one_key_model(size, dtype, dim, vdim, heads=2, kv_heads=1):
    """One windowed mixer without feed-forward whose queries are scaled up (through the norm's weights): the softmax
    is nearly one-hot, so a key that is wrongly seen or wrongly hidden changes the logits by much more than any
    tolerance."""
    sharp = 4.0 if dtype == "float32" else 2.5
    cfg = config(48, 61, [("attention", attention(heads, kv_heads, dim, vdim, 1.0, size, rot_dims=4, base=1e6), None)])
    w = pf.random_weights(cfg, seed=size * 31 + dim)
    w["l0.mix.q.norm"] = w["l0.mix.q.norm"] * sharp
    return cfg, cast(w, dtype)


def with_window(cfg, size):
    c = copy.deepcopy(cfg)
    c["layers"][0]["mixer"]["mask"] = dict(size=size)
    return c


EDGES = [(8, 32, 32), (4, 64, 64), (70, 64, 64), (5, 128, 128), (17, 24, 40), (9, 32, 48), (66, 128, 128), (33, 48, 16)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("size,dim,vdim", EDGES)
def test_window_edges_in_prompts_and_decoding(tmp_path, dtype, size, dim, vdim):
    page = 8
    cfg, w = one_key_model(size, dtype, dim, vdim)
    n = 70 if size < 40 else size + 40  # (long windows must pass over prompt and decoded tokens too)
    # the test has power: a window one token longer or shorter is far off (the first of a few token sequences for
    # which both are)
    others = [size + 1] + ([size - 1] if size > 1 else [])
    for seed in range(5, 25):
        ids = random_ids(cfg["vocab"], n, seed)
        ref = oracle(ids, w, cfg)
        offs = [float((oracle(ids, w, with_window(cfg, s)) - ref).abs().max() / ref.abs().max()) for s in others]
        if min(offs) > 5 * TOL[dtype]:
            break
    else:
        raise AssertionError(f"no token sequence makes every edge decisive (last: {offs})")
    r = make_runner(tmp_path, cfg, w, page, dtype, num_pages=14 if size < 40 else 20)
    # portions that end on, one before and one after page borders and window edges; then single tokens
    plan = [[("a", k)] for k in (7, 1, 1, 8, 9, 2, size, 3)]
    used = sum(k for (_, k), in plan)
    plan += [[("a", 1)] for _ in range(n - used)]
    got = replay(r, {"a": ids}, plan)["a"]
    what = f"window {size}, heads of {dim} / {vdim}"
    if dtype == "float32":
        assert_close(got, ref, dtype, what)
    else:
        # sharp queries multiply the rounding of the 16-bit queries and keys; the largest error stays a quarter of
        # what the nearest wrong edge would cause, the mean error inside the models' limit
        mx, rms = errors(got, ref)
        assert torch.isfinite(got.float()).all(), f"{what}: non-finite logits"
        assert mx <= max(TOL[dtype], min(offs) / 4) and rms <= TOL_RMS[dtype], (
            f"{what}: max err {mx:.3e} of scale (a wrong edge: {min(offs):.3e}), rms {rms:.3e}")
    assert all(r.cache.num_free_pages(g) == n for g, n in enumerate(r.cache.group_pages))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rank,rot", [(40, 8), (112, 16)])
def test_a_far_key_among_hundreds_decides(tmp_path, dtype, rank, rot):
    """The causal latent layer with sharp queries: at the end of 400 tokens the asking token's query matches the key
    of ONE marked token near the start, and the logits say which token stood there.  The query of the asking token
    is made to point at the marked token's unrotated key: W_q's unrotated rows are the key up-projection applied to
    the marked token's latent direction, so the score is large there and nowhere else."""
    H, d, dv = 2, 16, 12
    cfg = config(48, 61, [("latent_attention", latent(H, d, rot, dv, rank, 1.0, base=1e4), None)])
    w = pf.random_weights(cfg, seed=rank)
    g = torch.Generator().manual_seed(9)
    asks, marked, other = 58, 60, 59
    wd = {n: t.double() for n, t in w.items()}
    eps = cfg["norm"]["eps"]

    def latent_of(tok):
        h = pf.rms_norm(wd["embed"][tok:tok + 1], wd["l0.norm1"], eps)
        return pf.rms_norm((h @ wd["l0.mix.dkv"].T)[:, :rank], wd["l0.mix.dkv.norm"], eps)[0]

    # every head's unrotated query of the asking token = sharp * (W_uk c_marked) of that head, through a rank-one
    # W_q on the asking token's normed embedding; the rotated query rows are zero
    h_ask = pf.rms_norm(wd["embed"][asks:asks + 1], wd["l0.norm1"], eps)[0]
    k_marked = (wd["l0.mix.uk"] @ latent_of(marked)).reshape(H, d)
    sharp = 6.0 if dtype == "float32" else 3.0
    wq = torch.zeros(H, d + rot, 48, dtype=torch.float64)
    wq[:, :d] = sharp * k_marked[:, :, None] * h_ask[None, None, :] / float(h_ask @ h_ask) / float((k_marked * k_marked).sum(-1).mean()) * d
    w["l0.mix.q"] = wq.reshape(H * (d + rot), 48).float()
    w = cast(w, dtype)
    n = 400
    ids = [t % 58 for t in random_ids(61, n, 3)]
    ids[13] = marked
    ids[-1] = asks
    ref = oracle(ids, w, cfg)
    changed = list(ids)
    changed[13] = other
    assert (oracle(changed, w, cfg)[-1] - ref[-1]).abs().max() > 5 * TOL[dtype] * ref.abs().max(), "token 13 must matter"
    r = make_runner(tmp_path, cfg, w, 8, dtype, num_pages=56)
    plan = [[("a", 64)] for _ in range(5)] + [[("a", 2)] for _ in range(20)] + [[("a", 1)] for _ in range(40)]
    got = replay(r, {"a": ids}, plan)["a"]
    assert_close(got[-1:], ref[-1:], dtype, "far key, last row")
    assert_rows_close(got, ref, dtype, "far key")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_first_tokens_alone_and_in_pairs(tmp_path, dtype):
    """Requests of one, two and three tokens, each alone in a step and side by side: the first positions (angle 0, a
    softmax over one key, a window that is not full) against the plain model."""
    for tag in ("A", "B", "D"):
        cfg, w, page = model_for(tag, dtype)
        r = make_runner(tmp_path, cfg, w, page, dtype, name=tag)
        reqs = {k: random_ids(cfg["vocab"], n, 7 + n) for k, n in dict(a=1, b=2, c=3, d=2).items()}
        got = replay(r, reqs, [[("a", 1)], [("b", 2), ("c", 1)], [("c", 2), ("d", 1)], [("d", 1)]])
        for k in reqs:
            assert_rows_close(got[k], oracle(reqs[k], w, cfg), dtype, f"{tag} request {k}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(tmp_path, dtype):
    """One prompt token, then 300 tokens one by one: windows slide over decoded tokens, pages come and go, the
    loop's passes keep caches of their own."""
    cfg, w, page = model_for("B", dtype)
    r = make_runner(tmp_path, cfg, w, page, dtype, num_pages=160)
    ids = random_ids(cfg["vocab"], 301, 17)
    got = replay(r, {"a": ids}, [[("a", 1)] for _ in range(301)])["a"]
    assert_rows_close(got, oracle(ids, w, cfg), dtype, "long decoding")


# ---------------------------------------------------------------------------------------------------------
# generation through the entry point and the scheduler
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("eager", [True, False])
@pytest.mark.parametrize("tag", ["A", "C"])
def test_greedy_generation_through_the_entry_point(tmp_path, tag, eager):
    """Five prompts under a token budget of 16 and three request slots (prompts are cut into portions, requests
    wait for a slot, decode steps are replayed from CUDA graphs unless eager), greedy, against the plain model
    run on the growing sequence.  A step's choice is compared only where the plain model's margin is clear."""
    from ullm_b200 import LLM, EngineConfig, SamplingParams

    cfg, w, page = weights_for(tag, "float32")
    d = write_model(str(tmp_path / f"gen{tag}{eager}"), cfg, w)
    ec = EngineConfig(model=d, max_bs=3, context_len=128, page_size=page, num_pages=48, max_num_batched_tokens=16,
                      dtype="float32", enforce_eager=eager)
    llm = LLM(ec)
    prompts = [random_ids(cfg["vocab"], n, 90 + n) for n in (1, 6, 23, 40, 17)]
    outs = llm.generate_batch(prompts, SamplingParams(temperature=0.0, max_new_tokens=14, ignore_eos=True))
    wd = {n: t.double() for n, t in w.items()}
    for p, o in zip(prompts, outs):
        assert len(o.token_ids) == 14
        seq = list(p)
        for tok in o.token_ids:
            lg = pf.forward(cfg, wd, seq)[-1]
            top2 = torch.topk(lg, 2).values
            if top2[0] - top2[1] > 1e-3 * lg.abs().max():
                assert tok == int(torch.argmax(lg)), f"prompt of {len(p)}: token {len(seq) - len(p)} differs"
            seq.append(tok)
    llm.engine.runner.cache.check_invariants()
