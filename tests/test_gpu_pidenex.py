"""The Pidenex decoder in the engine against the plain implementation (tests/plain_pidenex.py): each mechanism
alone, whole prompts against token-by-token decoding and portions down to two tokens, unequal batches with pages
and state slots that are used again, the edges of windows and of pooled blocks (with weights made so that one key
decides), far memory of the recurrence, the first tokens, long decoding, and greedy generation through the entry
point and the scheduler."""

import copy

import pytest
import torch

import plain_pidenex as pp
from conftest import device
from helpers import TOL, TOL_RMS, assert_close, errors, random_ids
from ludalix_helpers import assert_rows_close
from pidenex_helpers import (CONFIGS, attention, cast, config, dense, latent, make_runner, oracle, parallel, replay,
                             weights_for, write_model)

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
    return [i for i, _ in pp.layer_runs(cfg)].index(layer)


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
    """Random rows in four steps (29, 2, 1 and 15 tokens: windows of 1 to 40 and blocks of 1 to 16 pass their
    edges inside a portion and between portions) against the mixer run whole."""
    cfg, w, page = weights_for(tag, dtype)
    r = make_runner(tmp_path, cfg, w, page, dtype)
    x = rand((47, cfg["width"]), 5 + layer, dtype)
    wd = {n: t.double() for n, t in w.items()}
    L = cfg["layers"][layer]
    ref = pp.mixer(L["type"], x.double().cpu(), L["mixer"], wd, f"l{layer}.mix.", cfg["norm"]["eps"]).float()
    got = mixer_in_steps(r, cfg, layer, x, (29, 31, 32))
    close(got, ref, dtype, f"{tag} layer {layer} ({L['type']})")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_two_branches_of_a_parallel_mixer_alone(tmp_path, dtype):
    """Each branch in front of the shared output product, with its scale: the biased, gated attention and the
    recurrence."""
    from ullm_b200.engine import StepEntry

    cfg, w, page = weights_for("A", dtype)
    r = make_runner(tmp_path, cfg, w, page, dtype)
    m = cfg["layers"][0]["mixer"]
    x = rand((33, cfg["width"]), 3, dtype)
    wd = {n: t.double() for n, t in w.items()}
    xd = x.double().cpu()
    left = m["left_scale"] * pp.biased_attention_unprojected(xd, m["left"], wd, "l0.mix.left.", cfg["norm"]["eps"])
    right = m["right_scale"] * pp.mingru_unprojected(xd, wd, "l0.mix.right.")[0]
    mixer = r.model.blocks[0].mixer
    got_l, got_r = [], []
    r.add_request("a")
    for a, b in ((0, 20), (20, 22), (22, 23), (23, 33)):
        e = [StepEntry("a", [0] * (b - a), [])]
        ctx = r.prepare(e)
        cache = r.cache.layer_caches(ctx.groups)[0]
        got_l.append(mixer.left.forward(x[a:b].clone(), ctx, cache, project_output=False,
                                        out_scale=m["left_scale"]).float().cpu().clone())
        got_r.append(mixer.right.forward(x[a:b].clone(), ctx, cache, project_output=False,
                                         out_scale=m["right_scale"]).float().cpu().clone())
        r.commit(e)
    r.check_device_status()
    close(torch.cat(got_l), left.float(), dtype, "left branch")
    close(torch.cat(got_r), right.float(), dtype, "right branch")


def test_candidate_and_gate_of_the_recurrence_take_both_branches():
    """The plain recurrence against its closed form S_t = sum_s z_s c_s prod_{s < r <= t} (1 - z_r), and the
    candidate on both sides of zero (continuous there: 1/2)."""
    g = torch.Generator().manual_seed(1)
    n, W, H = 19, 6, 10
    h = torch.randn(n, H, generator=g).double()
    w = {"z": torch.randn(W, H, generator=g).double(), "z.b": torch.randn(W, generator=g).double(),
         "x": torch.randn(W, H, generator=g).double(), "x.b": torch.randn(W, generator=g).double(),
         "g": torch.randn(W, H, generator=g).double()}
    out, S = pp.mingru_unprojected(h, w, "")
    z = torch.sigmoid(h @ w["z"].T + w["z.b"])
    u = h @ w["x"].T + w["x.b"]
    assert (u > 0).any() and (u < 0).any()
    c = torch.where(u >= 0, u + 0.5, 1 / (1 + torch.exp(-u)))
    ref = torch.zeros(W).double()
    for s in range(n):
        ref = ref + z[s] * c[s] * torch.prod(1 - z[s + 1:], 0)
    assert torch.allclose(S, ref, rtol=1e-10, atol=1e-12)
    gg = h[-1] @ w["g"].T
    assert torch.allclose(out[-1], ref * gg / (1 + torch.exp(-gg)), rtol=1e-10, atol=1e-12)
    assert abs(float(torch.where(torch.tensor(0.0) >= 0, torch.tensor(0.5), torch.tensor(0.0))) - 0.5) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_and_its_activation_alone(tmp_path, dtype):
    from ullm_b200.engine.batch import Workspace

    for tag, layers in (("A", (0, 2)), ("C", (0, 1, 2))):
        cfg, w, page = weights_for(tag, dtype)
        # both numbers of the activation away from their start, the second branch steep
        for l in layers:
            w[f"l{l}.mlp.act"] = torch.tensor([0.7 - l, -0.4 + 0.9 * l]).to(w[f"l{l}.mlp.act"].dtype)
        r = make_runner(tmp_path, cfg, w, page, dtype, name=tag)

        class Ctx:
            workspace = Workspace(r.device, max_tokens=32, max_requests=4)

        x = rand((21, cfg["width"]), 8, dtype, 1.5)
        wd = {k: t.double() for k, t in w.items()}
        for l in layers:
            ref = pp.dense_ff(x.double().cpu(), wd, f"l{l}.mlp.").float()
            close(r.model.blocks[l].feed_forward.forward(x.clone(), Ctx()), ref, dtype, f"{tag} layer {l} feed-forward")


def test_pooled_blocks_and_slopes_in_the_plain_attention_core():
    """The plain core against a direct evaluation: query 13 under a window of 5 with blocks of 3 sees the tokens
    9 .. 13 and the blocks 0, 1, 2 (block 2 ends at 8 = 13 - 5); query 12 sees two blocks and the tokens 8 .. 12,
    token 6 and 7 not at all.  Slopes: head h of H loses 2^(-8 (h + 1) / H) per position of distance."""
    g = torch.Generator().manual_seed(4)
    q, k = torch.randn(2, 14, 4, generator=g).double(), torch.randn(1, 14, 4, generator=g).double()
    out = pp.window_attention(q, k, k, 0.5, 5, pool=3).reshape(14, 2, 4)
    for i, blocks, lo in ((13, 3, 9), (12, 2, 8), (4, 0, 0), (7, 1, 3)):
        keys = [k[0, b * 3:b * 3 + 3].mean(0) for b in range(blocks)] + [k[0, j] for j in range(lo, i + 1)]
        K = torch.stack(keys)
        for h in range(2):
            p = torch.softmax(K @ q[h, i] * 0.5, 0)
            assert torch.allclose(out[i, h], p @ K, rtol=1e-10, atol=1e-12), (i, h)
    s = pp.head_slopes(4, torch.float64)
    assert torch.allclose(s, torch.tensor([0.25, 0.0625, 2.0 ** -6, 2.0 ** -8]).double())
    out = pp.window_attention(q, k, k, 0.5, 4, slopes=pp.head_slopes(2, torch.float64)).reshape(14, 2, 4)
    for h in range(2):
        sc = torch.stack([k[0, j] @ q[h, 9] * 0.5 - 2.0 ** (-4 * (h + 1)) * (9 - j) for j in range(6, 10)])
        assert torch.allclose(out[9, h], torch.softmax(sc, 0) @ k[0, 6:10], rtol=1e-10, atol=1e-12)


# ---------------------------------------------------------------------------------------------------------
# whole prompts, token-by-token decoding, portions
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "B", "C", "D", "E"])
def test_whole_decode_and_portions_agree_with_the_plain_model(tmp_path, dtype, tag):
    cfg, w, page = weights_for(tag, dtype)
    r = make_runner(tmp_path, cfg, w, page, dtype, num_pages=96 if tag == "B" else 64)
    n = 75 if tag != "E" else 150  # (E: the windows of 70 and 90 must pass over prompt and decoded tokens)
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
    """Three state slots and a pool that cannot hold all requests at once: six requests of unequal length come
    and go, portions of some beside single tokens of others; every request equals itself run alone."""
    cfg, w, page = weights_for(tag, dtype)
    pages = 22 if tag == "A" else 17
    r = make_runner(tmp_path, cfg, w, page, dtype, num_pages=pages, max_requests=3)
    lens = dict(a=50, b=9, c=61, d=2, e=33, f=17)
    reqs = {k: random_ids(cfg["vocab"], n, 40 + n) for k, n in lens.items()}
    plan = [
        [("a", 20), ("b", 2)],
        [("a", 1), ("b", 5), ("c", 30)],
        [("b", 2), ("a", 9), ("c", 1)],          # b ends: its slot and pages go back
        [("d", 2), ("c", 1), ("a", 1)],          # d takes them, and ends at once
        [("e", 16), ("a", 19)],                  # a ends
        [("c", 29), ("e", 1), ("f", 2)],         # c ends; f starts on a slot that held state
        [("f", 15), ("e", 16)],
    ]
    got = replay(r, reqs, plan)
    for k in reqs:
        assert_rows_close(got[k], oracle(reqs[k], w, cfg), dtype, f"request {k}")
    assert not r.cache.requests
    assert all(r.cache.num_free_pages(g) == n for g, n in enumerate(r.cache.group_pages))


# ---------------------------------------------------------------------------------------------------------
# edges: windows, pooled blocks, page borders; weights made so that one key decides
# ---------------------------------------------------------------------------------------------------------
def one_key_model(kind, size, pool, dtype, dim):
    """One mixer without feed-forward whose queries are scaled up: the softmax is nearly one-hot, so a key or a
    block that is wrongly seen or wrongly hidden changes the logits by much more than any tolerance."""
    sharp = 4.0 if dtype == "float32" else 2.5
    if kind == "attention":
        m = attention(2, 1, dim, 1.0, size, pool=pool)
        grow = ["l0.mix.q"]
    elif kind == "parallel":
        m = parallel(2, 1, dim, 1.0, size, 16, 1.0, 0.2)
        grow = ["l0.mix.left.q.norm"]
    else:
        # (scores grow with the rank: the scale keeps the sharpness of the small ranks)
        rot = 64 if dim in (384, 512) else 16  # (key rows of 384 + 64 and 512 + 64: sizes the kernel knows as constants)
        m = latent(2, dim, rot, 24, dim, 24, min(1.0, 48.0 / dim), size, base=50.0)
        grow = ["l0.mix.uq"]
    cfg = config(48, 61, [(kind, m, None)], scale=3.0)
    w = pp.random_weights(cfg, seed=size * 31 + pool)
    for n in grow:
        w[n] = w[n] * sharp
    return cfg, cast(w, dtype)


def with_mask(cfg, size, pool):
    c = copy.deepcopy(cfg)
    m = c["layers"][0]["mixer"]
    m = m["left"] if c["layers"][0]["type"] == "parallel" else m
    m["mask"] = dict(size=size, **({"pool": pool} if pool else {}))
    return c


EDGES = [("attention", 8, 4, 32), ("attention", 4, 4, 64), ("attention", 70, 2, 64), ("attention", 5, 3, 128), ("attention", 17, 1, 24),
         ("attention", 9, 0, 64), ("parallel", 8, 0, 32), ("parallel", 17, 0, 64), ("latent_attention", 8, 0, 32),
         ("latent_attention", 19, 0, 48), ("parallel", 66, 0, 128), ("latent_attention", 67, 0, 160),
         ("latent_attention", 65, 0, 272), ("latent_attention", 21, 0, 400),
         ("latent_attention", 66, 0, 384), ("latent_attention", 33, 0, 512)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind,size,pool,dim", EDGES)
def test_window_and_block_edges_in_prompts_and_decoding(tmp_path, dtype, kind, size, pool, dim):
    page = 8
    cfg, w = one_key_model(kind, size, pool, dtype, dim)
    n = 70 if size < 40 else size + 40  # (long windows must pass over prompt and decoded tokens too)
    # the test has power: a window one token longer or shorter, or blocks one token longer or shorter, is far off
    # (the first of a few token sequences for which all are)
    # (blocks of one token are the tokens themselves: the window's size then changes nothing)
    others = ([(size + 1, pool), (size - 1, pool)] if pool != 1 else []) + (
        [(size, pool + 1)] + ([(size, pool - 1)] if pool > 1 else []) if pool else [])
    others = [o for o in others if o[0] > 0]
    for seed in range(5, 25):
        ids = random_ids(cfg["vocab"], n, seed)
        ref = oracle(ids, w, cfg)
        offs = [float((oracle(ids, w, with_mask(cfg, s, p)) - ref).abs().max() / ref.abs().max()) for s, p in others]
        if min(offs) > 5 * TOL[dtype]:
            break
    else:
        raise AssertionError(f"no token sequence makes every edge decisive (last: {offs})")
    r = make_runner(tmp_path, cfg, w, page, dtype, num_pages=14)
    # portions that end on, one before and one after page borders, window edges and block ends; then single tokens
    plan = [[("a", k)] for k in (7, 1, 1, 8, 9, 2, size, 3)]
    used = sum(k for (_, k), in plan)
    plan += [[("a", 1)] for _ in range(n - used)]
    got = replay(r, {"a": ids}, plan)["a"]
    what = f"{kind}: window {size}, blocks of {pool}"
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
def test_a_far_block_among_hundreds_of_keys_decides(tmp_path, dtype):
    """Blocks of 4 behind a window of 12 with sharp queries: at the end of 400 tokens a query still finds the one
    block near the start that matches it.  Values are keys, and a token's sharp query finds its own key first; so
    the asking token's query is made to point at ANOTHER token's key: the embeddings of the two are mirror images
    under a reflection S (zero mean, equal length, so the norm keeps them so), and W_q = sharp W_k S."""
    cfg, w = one_key_model("attention", 12, 4, "float32", 32)
    g = torch.Generator().manual_seed(9)
    width = cfg["width"]
    u, v = torch.randn(width, generator=g), torch.randn(width, generator=g)
    u, v = u - u.mean(), v - v.mean()
    v = v - (v @ u) / (u @ u) * u
    u, v = u / u.norm(), v / v.norm()
    asks, marked, other = 58, 60, 59
    w["embed"][asks], w["embed"][marked] = u, v
    w["l0.norm1"] = torch.ones(width)
    d = (u - v).unsqueeze(1)
    S = torch.eye(width) - 2 * (d @ d.T) / float(d.T @ d)
    sharp = 4.0 if dtype == "float32" else 2.5
    w["l0.mix.q"] = sharp * torch.cat([w["l0.mix.k"] @ S] * 2)
    w = cast(w, dtype)
    n = 400
    ids = [t % 58 for t in random_ids(61, n, 3)]
    ids[12:16] = [marked] * 4
    ids[-1] = asks
    ref = oracle(ids, w, cfg)
    changed = list(ids)
    changed[12:16] = [other] * 4
    assert (oracle(changed, w, cfg)[-1] - ref[-1]).abs().max() > 5 * TOL[dtype] * ref.abs().max(), "block 3 must matter"
    r = make_runner(tmp_path, cfg, w, 8, dtype, num_pages=56)
    plan = [[("a", 64)] for _ in range(5)] + [[("a", 2)] for _ in range(20)] + [[("a", 1)] for _ in range(40)]
    got = replay(r, {"a": ids}, plan)["a"]
    assert_close(got, ref, dtype, "far block")


def test_the_recurrence_remembers_far_tokens(tmp_path):
    """Update gates that stay nearly shut except for one marked token (its embedding points along the gate's
    weight): what the token at position 2 wrote dominates the state two hundred tokens later, through portions,
    decoding and a slot that held another request's state before."""
    cfg = config(40, 53, [("parallel", parallel(2, 1, 16, 0.25, 6, 24, 0.1, 1.5), None),
                          ("parallel", parallel(1, 1, 16, 0.25, 4, 40, 0.1, 1.0), dense(48))], scale=2.0)
    w = pp.random_weights(cfg, seed=21)
    g = torch.Generator().manual_seed(4)
    u = torch.nn.functional.normalize(torch.randn(40, generator=g), dim=0)
    marked = (51, 52)
    for z in marked:
        w["embed"][z] = (40.0 * u + 12.0 * torch.nn.functional.normalize(torch.randn(40, generator=g), dim=0)) / 2.0
    w["l0.mix.right.z"] = 2.0 * (u - u.mean()).repeat(24, 1)
    for l in (0, 1):
        w[f"l{l}.mix.right.z.b"] = torch.full_like(w[f"l{l}.mix.right.z.b"], -6.0)
    w["l1.mix.right.z"] = w["l1.mix.right.z"] * 0.05
    n = 230
    ids = [t % 51 for t in random_ids(53, n, 13)]
    ids[2] = marked[0]
    ref = oracle(ids, w, cfg)
    changed = list(ids)
    changed[2] = marked[1]
    assert (oracle(changed, w, cfg)[-20:] - ref[-20:]).abs().max() > 5 * TOL["float32"] * ref.abs().max(), (
        "token 2 must matter at the end")
    r = make_runner(tmp_path, cfg, w, 16, "float32", num_pages=32, max_requests=2)
    got = replay(r, {"x": changed[:40], "a": ids}, [
        [("x", 40)],                                  # leaves state in slot 0, which "a" then takes
        [("a", 3)], [("a", 60)], [("a", 64)], [("a", 2)], [("a", 61)]] + [[("a", 1)] for _ in range(40)])
    assert_close(got["a"], ref, "float32", "far memory")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(tmp_path, dtype):
    """One prompt token, then 300 tokens one by one: windows slide over decoded tokens, blocks fill, pages come and
    go, the loop's passes keep caches of their own."""
    cfg, w, page = weights_for("B", dtype)
    r = make_runner(tmp_path, cfg, w, page, dtype, num_pages=120)
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
            lg = pp.forward(cfg, wd, seq)[-1]
            top2 = torch.topk(lg, 2).values
            if top2[0] - top2[1] > 1e-3 * lg.abs().max():
                assert tok == int(torch.argmax(lg)), f"prompt of {len(p)}: token {len(seq) - len(p)} differs"
            seq.append(tok)
    llm.engine.runner.cache.check_invariants()
