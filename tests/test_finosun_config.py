"""Host-side pieces of the Finosun decoder that need no GPU: the config.json reader, the tensor names the model
declares, the layer runs a loop unrolls into, what the cache manager plans for its mixers and passes, and the plain
implementation's own reading of each mechanism."""

import copy

import pytest
import torch

import plain_finosun as pf
from finosun_helpers import CFG_A, CFG_B, CFG_C, CFG_D, CFG_E, attention, config, latent, moe


def _spec(cfg):
    from ullm_b200.config import load_model_spec

    return load_model_spec(copy.deepcopy(cfg))[1]


def _shapes(cfg):
    return {n: tuple(s) for n, (s, _) in pf.tensor_shapes(cfg).items()}


def test_the_model_declares_exactly_the_checkpoints_tensors():
    from ullm_b200.parts.model import DecoderModel

    for cfg in (CFG_A, CFG_B, CFG_C, CFG_D, CFG_E):
        spec = _spec(cfg)
        model = DecoderModel(spec)
        assert {n: tuple(d.shape) for n, d in model.all_decls().items()} == _shapes(cfg)
        assert spec.stream_dtype == "float32" and spec.tie_embeddings


def test_a_loop_unrolls_into_runs_with_the_projection_at_the_first_layer_of_each_pass():
    for cfg in (CFG_A, CFG_B, CFG_C, CFG_D, CFG_E):
        spec = _spec(cfg)
        runs = pf.layer_runs(cfg)
        assert [e.layer for e in spec.schedule] == [i for i, _ in runs]
        assert [e.project_input for e in spec.schedule] == [s for _, s in runs]
        assert all(e.cache_of is None for e in spec.schedule)  # every pass keeps a cache of its own
        assert (spec.pass_projection == "loop.in") == ("loop" in cfg)
    assert len(_spec(CFG_A).schedule) == 1 + 2 * 2 and len(_spec(CFG_B).schedule) == 6
    assert [s for _, s in pf.layer_runs(CFG_B)] == [True, False] * 3  # the first pass starts with it too
    assert [s for _, s in pf.layer_runs(CFG_D)] == [False, False, True, False, False]


def test_allocated_tensors_have_the_declared_names_and_32_bit_where_the_arithmetic_is():
    from ullm_b200.parts.model import DecoderModel

    model = DecoderModel(_spec(CFG_A))
    model.allocate("cpu", torch.bfloat16)
    t = model.all_tensors()
    assert {n: tuple(v.shape) for n, v in t.items()} == _shapes(CFG_A)
    for n, v in t.items():
        last = n.split(".")[-1]
        is32 = last.startswith("norm") or last in ("ls1", "ls2", "temp", "correction")
        assert v.dtype == (torch.float32 if is32 else torch.bfloat16), n


@pytest.mark.parametrize("change,needle", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].update(eps=0), "eps"),
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=26), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(base=0), "base"),
    (lambda c: c["layers"][0]["mixer"]["mask"].pop("size"), "size"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=8), "rot_dim"),
    (lambda c: c["layers"][1]["mixer"].update(rot_dim=-2), "rot_dim"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=8), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(identity=-1), "identity"),
    (lambda c: c["layers"][0]["mlp"]["shared"].pop("ff"), "ff"),
    (lambda c: c["loop"].update(stop=4), "loop"),
    (lambda c: c["loop"].update(times=0), "times"),
])
def test_config_errors_name_the_key(change, needle):
    from ullm_b200.config import load_model_spec
    from ullm_b200.config.finosun import FinosunConfigError

    cfg = copy.deepcopy(CFG_A)
    change(cfg)
    with pytest.raises(FinosunConfigError, match=needle):
        load_model_spec(cfg)


def test_every_pass_gets_pages_of_its_own_and_each_mixer_the_cache_it_needs():
    from ullm_b200.cache.manager import plan_groups_with_aux
    from ullm_b200.parts.model import DecoderModel

    needs = DecoderModel(_spec(CFG_A)).cache_needs()  # runs: window | latent, window | latent, window
    assert len(needs) == 5
    groups, where, where_aux = plan_groups_with_aux(needs)
    assert all(w is not None for w in where) and len(set(where)) == 5 and all(a is None for a in where_aux)
    # the windowed layers keep keys and values of their own widths, and give pages behind the window back
    assert (needs[0][0].num_kv_heads, needs[0][0].head_dim, needs[0][0].v_dim, needs[0][0].window) == (2, 24, 40, 9)
    assert (needs[2][0].num_kv_heads, needs[2][0].head_dim, needs[2][0].v_dim, needs[2][0].window) == (1, 16, 16, 13)
    # the latent layers keep ONE row [latent | rotated part] per token, and every token
    assert needs[1][0].values_in_keys and (needs[1][0].num_kv_heads, needs[1][0].head_dim) == (1, 40 + 12)
    assert needs[1][0].window is None
    # the two passes share a group (equal needs) but not their pages; nothing has per-request state
    assert where[1][0] == where[3][0] and where[2][0] == where[4][0] and where[1] != where[3] and where[2] != where[4]
    assert all(n[1] is None for n in needs)


# ---------------------------------------------------------------------------------------------------------
# the plain implementation's own reading of each mechanism, against direct evaluations
# ---------------------------------------------------------------------------------------------------------
def test_the_two_rotations_pair_neighbours_and_halves():
    g = torch.Generator().manual_seed(2)
    v = torch.randn(3, 10, generator=g).double()
    pos = torch.tensor([0, 5, 11])
    a = pf.rotate_neighbours(v, pos, 6, 100.0)
    b = pf.rotate_halves(v, pos, 6, 100.0)
    for t, p in enumerate(pos.tolist()):
        for i in range(3):
            ang = p * 100.0 ** (-2.0 * i / 6)
            c, s = torch.cos(torch.tensor(ang).double()), torch.sin(torch.tensor(ang).double())
            assert torch.allclose(a[t, 2 * i], v[t, 2 * i] * c - v[t, 2 * i + 1] * s)
            assert torch.allclose(a[t, 2 * i + 1], v[t, 2 * i + 1] * c + v[t, 2 * i] * s)
            assert torch.allclose(b[t, i], v[t, i] * c - v[t, i + 3] * s)
            assert torch.allclose(b[t, i + 3], v[t, i + 3] * c + v[t, i] * s)
    assert torch.equal(a[:, 6:], v[:, 6:]) and torch.equal(b[:, 6:], v[:, 6:]) and torch.allclose(a[0], v[0])


def test_the_window_sees_itself_and_size_minus_one_tokens_before():
    g = torch.Generator().manual_seed(4)
    q, k, v = (torch.randn(2, 9, 4, generator=g).double() for _ in range(3))
    out = pf.masked_attention(q, k[:1], v[:1], torch.tensor([0.5, 2.0]).double(), 3).reshape(9, 2, 4)
    for i, lo in ((0, 0), (1, 0), (2, 0), (3, 1), (8, 6)):
        for h, f in ((0, 0.5), (1, 2.0)):
            p = torch.softmax(k[0, lo:i + 1] @ q[h, i] * f, 0)
            assert torch.allclose(out[i, h], p @ v[0, lo:i + 1], rtol=1e-10, atol=1e-12)
    whole = pf.masked_attention(q, k[:1], v[:1], torch.ones(2).double(), None).reshape(9, 2, 4)
    assert torch.allclose(whole[8, 1], torch.softmax(k[0] @ q[1, 8], 0) @ v[0], rtol=1e-10, atol=1e-12)


def test_the_choice_takes_the_correction_and_the_weight_does_not():
    w = {"router": torch.eye(4).double(), "correction": torch.tensor([0.0, 0.0, 0.0, 10.0]).double()}
    h = torch.tensor([[3.0, 2.0, 1.0, 0.0]]).double()
    chosen, weight = pf.route(h, w, "", 2)
    s = torch.softmax(h[0], 0)
    assert chosen.tolist() == [[3, 0]]  # the corrected output first, then the largest score
    assert torch.allclose(weight[0], torch.stack([s[3], s[0]]))  # the scores themselves, not renormalized
    assert float(weight.sum()) < 1.0


def test_passing_experts_and_the_shared_expert_in_the_plain_feed_forward():
    cfg = config(8, 11, [("attention", attention(1, 1, 4, 4, 0.5, 2), moe(2, 1, 3, 4, 0.7, shared=(4, 0.9)))])
    w = {n: t.double() for n, t in pf.random_weights(cfg, seed=3).items()}
    f, pre = cfg["layers"][0]["mlp"], "l0.mlp."
    h = torch.randn(5, 8, generator=torch.Generator().manual_seed(1)).double()
    s = torch.softmax(h @ w[pre + "router"].T, -1)
    ref = s[:, 2:3] * h  # every output is chosen: the third one passes the input
    for e in range(2):
        g = torch.clamp(h @ w[f"{pre}e{e}.gate"].T, max=0.7)
        u = torch.clamp(h @ w[f"{pre}e{e}.up"].T, -0.7, 0.7)
        ref = ref + s[:, e:e + 1] * ((g * torch.sigmoid(1.702 * g) * (u + 1)) @ w[f"{pre}e{e}.down"].T)
    g = torch.clamp(h @ w[pre + "shared.gate"].T, max=0.9)
    u = torch.clamp(h @ w[pre + "shared.up"].T, -0.9, 0.9)
    ref = ref + torch.sigmoid(h @ w[pre + "shared.sg"].T) * ((g * torch.sigmoid(1.702 * g) * (u + 1)) @ w[pre + "shared.down"].T)
    assert torch.allclose(pf.routed_ff(h, f, w, pre), ref, rtol=1e-10, atol=1e-12)


def test_the_latent_scores_equal_the_absorbed_form():
    """(q_plain . W_uk c + q_rot . k_rot) = (W_uk^T q_plain) . c + q_rot . k_rot: what lets a cache hold [c | k_rot]."""
    cfg = config(16, 11, [("latent_attention", latent(2, 6, 4, 5, 7, 0.3, base=9.0), None)])
    w = {n: t.double() for n, t in pf.random_weights(cfg, seed=5).items()}
    m, pre = cfg["layers"][0]["mixer"], "l0.mix."
    h = torch.randn(6, 16, generator=torch.Generator().manual_seed(2)).double()
    pos = torch.arange(6)
    down = h @ w[pre + "dkv"].T
    c = pf.rms_norm(down[:, :7], w[pre + "dkv.norm"], 2e-6)
    kr = pf.rotate_halves(down[:, 7:], pos, 4, 9.0)
    q = (h @ w[pre + "q"].T).reshape(6, 2, 10)
    out = torch.zeros(6, 2, 5).double()
    for hd in range(2):
        uk, uv = w[pre + "uk"][hd * 6:(hd + 1) * 6], w[pre + "uv"][hd * 5:(hd + 1) * 5]
        qa = q[:, hd, :6] @ uk  # absorbed: [n, rank]
        qr = pf.rotate_halves(q[:, hd, 6:], pos, 4, 9.0)
        for i in range(6):
            sc = (c[:i + 1] @ qa[i] + kr[:i + 1] @ qr[i]) * 0.3
            out[i, hd] = (torch.softmax(sc, 0) @ c[:i + 1]) @ uv.T
    ref = (out.reshape(6, 10) * torch.sigmoid(h @ w[pre + "g"].T)) @ w[pre + "o"].T
    assert torch.allclose(pf.latent_attention(h, m, w, pre, 2e-6), ref, rtol=1e-9, atol=1e-11)
