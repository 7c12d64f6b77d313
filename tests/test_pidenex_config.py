"""Host-side pieces of the Pidenex decoder that need no GPU: the config.json reader, the tensor names the model
declares, the layer runs a loop unrolls into, what the cache manager plans for windows with pooled blocks behind
them and for passes with caches of their own, and the plain implementation's own reading of each mechanism."""

import copy
import math

import pytest
import torch

import plain_pidenex as pp
from pidenex_helpers import CFG_A, CFG_B, CFG_C, CFG_D, attention, config, dense, latent, parallel


def _spec(cfg):
    from ullm_b200.config import load_model_spec

    return load_model_spec(copy.deepcopy(cfg))[1]


def test_the_model_declares_exactly_the_checkpoints_tensors():
    from ullm_b200.parts.model import DecoderModel

    for cfg in (CFG_A, CFG_B, CFG_C, CFG_D):
        spec = _spec(cfg)
        model = DecoderModel(spec)
        got = {n: tuple(d.shape) for n, d in model.all_decls().items()}
        assert got == pp.tensor_shapes(cfg)
        assert spec.stream_dtype == "float32" and spec.embedding_scale == cfg["embedding"]["scale"]


def test_a_loop_unrolls_into_runs_with_the_pass_vector_at_the_first_layer_of_each_pass():
    for cfg in (CFG_A, CFG_B, CFG_C, CFG_D):
        spec = _spec(cfg)
        runs = pp.layer_runs(cfg)
        assert [e.layer for e in spec.schedule] == [i for i, _ in runs]
        assert [e.add_vector for e in spec.schedule] == [t for _, t in runs]
        # the embedding's output comes again before every pass but the first
        assert [bool(e.add_input) for e in spec.schedule] == [t is not None and t > 0 for _, t in runs]
        assert all(e.cache_of is None for e in spec.schedule)  # every pass keeps a cache of its own
    assert len(_spec(CFG_A).schedule) == 1 + 2 * 2 and len(_spec(CFG_B).schedule) == 9


def test_allocated_tensors_have_the_declared_names_and_32_bit_where_the_arithmetic_is():
    from ullm_b200.parts.model import DecoderModel

    model = DecoderModel(_spec(CFG_A))
    model.allocate("cpu", torch.bfloat16)
    t = model.all_tensors()
    assert {n: tuple(v.shape) for n, v in t.items()} == pp.tensor_shapes(CFG_A)
    for n, v in t.items():
        last = n.split(".")[-1]
        is32 = last.startswith("norm") or n.endswith((".z.b", ".x.b", "mlp.act")) or n == "loop.step"
        assert v.dtype == (torch.float32 if is32 else torch.bfloat16), n


@pytest.mark.parametrize("change,needle", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["embedding"].pop("scale"), "scale"),
    (lambda c: c["norm"].update(eps=0), "eps"),
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(vdim=8), "vdim"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(pool=4), "pool"),
    (lambda c: c["layers"][0]["mixer"].pop("right_scale"), "right_scale"),
    (lambda c: c["layers"][0]["mixer"]["right"].pop("width"), "width"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=14), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][2]["mixer"]["mask"].pop("size"), "size"),
    (lambda c: c["layers"][2]["mixer"]["mask"].update(pool=0), "pool"),
    (lambda c: c["layers"][2]["mlp"].update(kind="moe"), "kind"),
    (lambda c: c["loop"].update(stop=4), "loop"),
    (lambda c: c["loop"].update(times=0), "times"),
])
def test_config_errors_name_the_key(change, needle):
    from ullm_b200.config import load_model_spec
    from ullm_b200.config.pidenex import PidenexConfigError

    cfg = copy.deepcopy(CFG_A)
    change(cfg)
    with pytest.raises(PidenexConfigError, match=needle):
        load_model_spec(cfg)


def _needs(cfg):
    from ullm_b200.parts.model import DecoderModel

    return DecoderModel(_spec(cfg)).cache_needs()


def test_every_pass_gets_pages_and_state_of_its_own_and_pooled_blocks_a_second_cache():
    from ullm_b200.cache.manager import plan_groups_with_aux

    needs = _needs(CFG_A)  # runs: parallel | latent, pooled attention | latent, pooled attention
    assert len(needs) == 5
    groups, where, where_aux = plan_groups_with_aux(needs)
    assert all(w is not None for w in where) and len({w for w in where}) == 5
    # the left branch keeps normed keys and raw values apart; the others read their values out of the key rows
    assert needs[0][0].values_in_keys is False and needs[0][0].window == 9 and needs[0][0].v_dim == 24
    assert needs[1][0].values_in_keys and (needs[1][0].num_kv_heads, needs[1][0].head_dim) == (1, 40 + 12)
    assert needs[2][0].values_in_keys and needs[2][0].window == 11
    assert where[1][0] == where[3][0] and where[2][0] == where[4][0] and where[1] != where[3]
    # the recurrence's state: one 32-bit row as wide as the recurrence, only at the parallel layer
    assert needs[0][1].shape == (40,) and needs[0][1].dtype == torch.float32
    assert all(n[1] is None for n in needs[1:])
    # blocks of 4: one entry per 4 tokens, all kept, for each of the two passes
    assert where_aux[0] is None and where_aux[1] is None and where_aux[2] is not None
    assert where_aux[2][0] == where_aux[4][0] and where_aux[2] != where_aux[4]
    aux = groups[where_aux[2][0]].need
    assert aux.every == 4 and aux.window is None and aux.head_dim == 16


def test_a_block_longer_than_the_window_keeps_its_tokens_until_it_is_complete():
    cfg = config(32, 40, [("attention", attention(2, 1, 16, 0.25, 3, pool=8), None)])
    need = _needs(cfg)[0][0]
    assert need.window == 8


def test_pages_behind_window_and_block_go_back_while_the_pooled_entries_stay():
    from ullm_b200.cache import CacheManager

    cfg = config(32, 40, [("attention", attention(2, 1, 16, 0.25, 6, pool=4), None)])
    cm = CacheManager(_needs(cfg), page_size=4, num_pages=12, max_requests=2, max_pages_per_request=12)
    rc = cm.admit("a")
    main = next(g for g, info in enumerate(cm.groups) if info.need.every == 1)
    pooled = next(g for g, info in enumerate(cm.groups) if info.need.every == 4)
    for n in (3, 9, 1, 20, 1, 1, 2):
        cm.reserve(rc, n)
        cm.commit(rc, n)
        cm.check_invariants()
        held = [i for i, p in enumerate(rc.pages[main]) if p >= 0]
        first_needed = max(0, rc.num_tokens - 6 + 1) // 4
        assert all(i >= first_needed for i in held) and all(i in held for i in range(first_needed, -(-rc.num_tokens // 4)))
        entries = rc.num_tokens // 4
        assert sum(p >= 0 for p in rc.pages[pooled]) == -(-entries // 4)
    cm.release(rc)
    # (a cache with one entry per 4 tokens is given a quarter of the pages, and one more per request)
    assert cm.num_free_pages(main) == 12 and cm.num_free_pages(pooled) == 12 // 4 + 2


# ---------------------------------------------------------------------------------------------------------
# the plain implementation's own reading, pinned on cases small enough to do by hand
# ---------------------------------------------------------------------------------------------------------
def test_plain_window_and_pooled_blocks_see_what_the_definition_says():
    """One head, keys e_j scaled so that the softmax weights can be read back from the output: with values =
    one-hot rows the output at i IS the softmax weight vector over what i sees."""
    n, size, P = 14, 5, 3
    k = torch.zeros(1, n, n, dtype=torch.float64)
    v = torch.eye(n, dtype=torch.float64)[None]
    q = torch.zeros(1, n, n, dtype=torch.float64)
    out = pp.window_attention(q, k, v, 1.0, size, pool=P).reshape(n, n)
    for i in range(n):
        lo = max(0, i - size + 1)
        blocks = [b for b in range(n // P) if b * P + P - 1 <= i - size]
        seen = len(blocks) + (i - lo + 1)
        expect = torch.zeros(n, dtype=torch.float64)
        expect[lo:i + 1] = 1.0 / seen
        for b in blocks:
            expect[b * P:(b + 1) * P] += 1.0 / (seen * P)
        assert torch.allclose(out[i], expect, atol=1e-12), i
        # tokens between the last seen block and the window are not seen at all
        hidden = [j for j in range(lo) if j // P not in blocks]
        assert all(out[i, j] == 0 for j in hidden)
    # i = 9: the window is 5..9; block 0 (0..2) ends at 2 <= 4, block 1 (3..5) ends at 5 > 4: 3 and 4 are hidden
    assert out[9, 3] == 0 and out[9, 4] == 0 and out[9, 0] > 0


def test_plain_slopes_rotation_activation_and_recurrence():
    s = pp.head_slopes(4, torch.float64)
    assert torch.allclose(s, torch.tensor([0.25, 0.0625, 0.015625, 0.00390625], dtype=torch.float64))
    # the bias is slope * distance taken OFF the score: with equal keys a nearer key weighs more
    n = 6
    q = torch.ones(1, n, 2, dtype=torch.float64)
    k = torch.ones(1, n, 2, dtype=torch.float64)
    v = torch.eye(n, dtype=torch.float64)[None]
    o = pp.window_attention(q, k, v, 1.0, 4, slopes=torch.tensor([0.5], dtype=torch.float64)).reshape(n, n)
    w = torch.exp(-0.5 * torch.tensor([3.0, 2.0, 1.0, 0.0], dtype=torch.float64))
    assert torch.allclose(o[5, 2:6], w / w.sum(), atol=1e-12) and o[5, 1] == 0
    # neighbours turn together; dimensions from `dims` on stay
    x = torch.tensor([[1.0, 0.0, 1.0, 0.0, 7.0, 9.0]], dtype=torch.float64).repeat(3, 1)
    r = pp.rotate_pairs(x, torch.arange(3), 4, 100.0)
    assert torch.allclose(r[2, :2], torch.tensor([math.cos(2.0), math.sin(2.0)], dtype=torch.float64))
    assert torch.allclose(r[2, 2:4], torch.tensor([math.cos(0.2), math.sin(0.2)], dtype=torch.float64))
    assert torch.equal(r[:, 4:], x[:, 4:]) and torch.equal(r[0], x[0])
    # activation: continuous at 0 with slope 1/2, quadratic above
    pq = torch.tensor([0.3, -0.2], dtype=torch.float64)
    z = torch.tensor([-1e-7, 0.0, 1e-7, 2.0, -3.0], dtype=torch.float64)
    a = pp.xielu(z, pq)
    assert abs(a[0] + 0.5e-7) < 1e-12 and a[1] == 0 and abs(a[2] - 0.5e-7) < 1e-12
    assert abs(a[3] - (math.log1p(math.exp(0.3)) * 4 + 1.0)) < 1e-12
    assert abs(a[4] - ((0.5 + math.log1p(math.exp(-0.2))) * (math.exp(-3.0) + 2.0) - 1.5)) < 1e-12
    # recurrence: a gate of one half averages the state with the candidate; the candidate's two branches
    w = {"z": torch.zeros(2, 1), "z.b": torch.zeros(2), "x": torch.tensor([[1.0], [-1.0]]), "x.b": torch.zeros(2),
         "g": torch.ones(2, 1)}
    w = {"p." + k: t.double() for k, t in w.items()}
    h = torch.tensor([[2.0], [2.0]], dtype=torch.float64)
    out, S = pp.mingru_unprojected(h, w, "p.")
    c = torch.tensor([2.5, 1 / (1 + math.exp(2.0))], dtype=torch.float64)
    assert torch.allclose(S, 0.75 * c) and torch.allclose(out[0], 0.5 * c * 2.0 / (1 + math.exp(-2.0)))
    # carried state: two halves equal the whole
    h = torch.randn(9, 1, dtype=torch.float64)
    whole, _ = pp.mingru_unprojected(h, w, "p.")
    a, S = pp.mingru_unprojected(h[:4], w, "p.")
    b, _ = pp.mingru_unprojected(h[4:], w, "p.", S)
    assert torch.allclose(torch.cat([a, b]), whole)


def test_plain_model_adds_embedding_and_pass_vectors_where_a_pass_starts():
    cfg = config(16, 20, [("attention", attention(1, 1, 8, 0.3, 4), None),
                          ("attention", attention(2, 1, 8, 0.3, 4), dense(12))], loop=(1, 2, 3))
    w = {n: t.double() for n, t in pp.random_weights(cfg, seed=1).items()}
    ids = [3, 1, 4, 1, 5]
    logits, after = pp.forward(cfg, w, ids, return_layers=True)
    assert after.shape == (4, 5, 16)
    x0 = w["embed"][torch.tensor(ids)] * cfg["embedding"]["scale"]
    x = pp.layer(x0, 0, cfg, w)
    assert torch.allclose(x, after[0])
    for t in range(3):
        x = x + (x0 if t else 0) + w["loop.step"][t]
        x = pp.layer(x, 1, cfg, w)
        assert torch.allclose(x, after[1 + t])
    assert torch.allclose(logits, pp.layer_norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["head"].T)
