"""The Pidenex decoder restated plainly: one slow function per mechanism, whole sequences at once, any float
dtype (the tests run it in 64-bit on the weights as given).  It shares no code with the engine.

Notation: n tokens, positions 0 .. n-1; x [n, width]; a linear map is `x @ W.T` with W [out, in].
"""

from __future__ import annotations

import math

import torch

# constants the design fixes
SLOPE_EXPONENT = 8.0


# ---------------------------------------------------------------------------------------------------------
# norms, activation, rotation
# ---------------------------------------------------------------------------------------------------------
def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdim=True)
    d = x - mu
    var = (d * d).mean(-1, keepdim=True)
    return d / torch.sqrt(var + eps) * w


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def softplus(v):
    return torch.log1p(torch.exp(-v.abs())) + torch.clamp(v, min=0)


def xielu(z, pq):
    """z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z / 2."""
    ap, aq = softplus(pq[0]), 0.5 + softplus(pq[1])
    neg = torch.clamp(z, max=0)
    return torch.where(z > 0, ap * z * z + 0.5 * z, aq * (torch.expm1(neg) - neg) + 0.5 * z)


def rotate_pairs(v, positions, dims, base):
    """v [..., n, d]: neighbours (2i, 2i+1), i < dims / 2, turn by the angle position * base^(-2i / dims); the
    dimensions from `dims` on stay."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims).to(v.dtype)
    a = positions.to(v.dtype)[:, None] * f[None, :]
    c, s = torch.cos(a), torch.sin(a)
    u, w = v[..., 0:dims:2], v[..., 1:dims:2]
    out = v.clone()
    out[..., 0:dims:2] = u * c - w * s
    out[..., 1:dims:2] = w * c + u * s
    return out


# ---------------------------------------------------------------------------------------------------------
# attention cores (scores in a loop over query positions: slow and plain)
# ---------------------------------------------------------------------------------------------------------
def mask_of(m):
    """(window size or None, pool or 0) of a mixer's configuration."""
    mk = m.get("mask")
    return (None, 0) if mk is None else (mk["size"], int(mk.get("pool") or 0))


def window_attention(q, k, v, scale, size, slopes=None, pool=0):
    """q [H, n, d], k [G, n, d], v [G, n, dv] -> [n, H * dv].  Query i sees j with 0 <= i - j < size (None: every
    j <= i); with `pool`
    P > 0 also one mean key / value per block of P positions that ends at or before i - size; with `slopes` [H]
    the score of (i, j) loses slopes[h] * (i - j).  One softmax over everything a query sees."""
    H, n, _ = q.shape
    G, dv = k.shape[0], v.shape[-1]
    rep = H // G
    size = n + 1 if size is None else size
    out = torch.zeros(n, H, dv, dtype=q.dtype)
    if pool:
        nb = n // pool
        kp = k[:, :nb * pool].reshape(G, nb, pool, k.shape[-1]).mean(2)
        vp = v[:, :nb * pool].reshape(G, nb, pool, dv).mean(2)
    for i in range(n):
        lo = max(0, i - size + 1)
        seen = (i - size + 1) // pool if (pool and i - size + 1 > 0) else 0  # blocks 0 .. seen-1 end before lo
        for h in range(H):
            g = h // rep
            s = (k[g, lo:i + 1] @ q[h, i]) * scale
            if slopes is not None:
                s = s - slopes[h] * (i - torch.arange(lo, i + 1)).to(q.dtype)
            vals = v[g, lo:i + 1]
            if seen:
                s = torch.cat([(kp[g, :seen] @ q[h, i]) * scale, s])
                vals = torch.cat([vp[g, :seen], vals])
            p = torch.softmax(s, 0)
            out[i, h] = p @ vals
    return out.reshape(n, H * dv)


def head_slopes(H, dtype):
    return torch.tensor([2.0 ** (-SLOPE_EXPONENT * (h + 1) / H) for h in range(H)], dtype=dtype)


# ---------------------------------------------------------------------------------------------------------
# mixers
# ---------------------------------------------------------------------------------------------------------
def latent_attention(h, m, w, pre, eps):
    """Queries and keys / values through low-rank latents; one rotated key part shared by the heads."""
    n = h.shape[0]
    H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(n)
    cq = rms_norm(h @ w[pre + "dq"].T, w[pre + "dq.norm"], eps)
    q = (cq @ w[pre + "uq"].T).reshape(n, H, d + r).transpose(0, 1)  # [H, n, d + r]
    dkv = h @ w[pre + "dkv"].T
    c = rms_norm(dkv[:, :R], w[pre + "dkv.norm"], eps)
    if not r:
        m = dict(m, rot=dict(dims=0, base=1.0))
    k_rot = rotate_pairs(dkv[:, R:], pos, m["rot"]["dims"], m["rot"]["base"])  # [n, r]
    k_plain = (c @ w[pre + "uk"].T).reshape(n, H, d).transpose(0, 1)
    v = (c @ w[pre + "uv"].T).reshape(n, H, dv).transpose(0, 1)
    q_rot = rotate_pairs(q[..., d:], pos, m["rot"]["dims"], m["rot"]["base"])
    qq = torch.cat([q[..., :d], q_rot], -1)
    kk = torch.cat([k_plain, k_rot[None].expand(H, n, r)], -1)
    size, pool = mask_of(m)
    o = window_attention(qq, kk, v, m["scale"], size, pool=pool)
    return o @ w[pre + "o"].T


def pooled_attention(h, m, w, pre):
    """Grouped heads, the keys are also the values, no positions, a window plus pooled blocks behind it."""
    n = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[pre + "q"].T).reshape(n, H, d).transpose(0, 1)
    k = (h @ w[pre + "k"].T).reshape(n, G, d).transpose(0, 1)
    size, pool = mask_of(m)
    o = window_attention(q, k, k, m["scale"], size, pool=pool)
    return o @ w[pre + "o"].T


def biased_attention_unprojected(h, m, w, pre, eps):
    """The left branch in front of its output map: the values are the keys before their norm; q and k are normed
    over the whole projection; scores lose slope_h * distance; the heads are gated by sigmoid(W_g h)."""
    n = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q_flat, k_flat = h @ w[pre + "q"].T, h @ w[pre + "k"].T
    v = k_flat.reshape(n, G, d).transpose(0, 1)
    q = rms_norm(q_flat, w[pre + "q.norm"], eps).reshape(n, H, d).transpose(0, 1)
    k = rms_norm(k_flat, w[pre + "k.norm"], eps).reshape(n, G, d).transpose(0, 1)
    o = window_attention(q, k, v, m["scale"], mask_of(m)[0], slopes=head_slopes(H, h.dtype))
    return o * torch.sigmoid(h @ w[pre + "g"].T)


def mingru_unprojected(h, w, pre, state=None):
    """S_t = (1 - z_t) S_{t-1} + z_t c_t per channel, S_0 = 0; returns (S_t * silu(W_g h_t) for every t, S_n)."""
    z = torch.sigmoid(h @ w[pre + "z"].T + w[pre + "z.b"])
    u = h @ w[pre + "x"].T + w[pre + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    g = h @ w[pre + "g"].T
    S = torch.zeros(z.shape[1], dtype=h.dtype) if state is None else state
    out = []
    for t in range(h.shape[0]):
        S = (1 - z[t]) * S + z[t] * cand[t]
        out.append(S * g[t] * torch.sigmoid(g[t]))
    return torch.stack(out), S


def parallel_mixer(h, m, w, pre, eps):
    left = biased_attention_unprojected(h, m["left"], w, pre + "left.", eps) @ w[pre + "left.o"].T
    right = mingru_unprojected(h, w, pre + "right.")[0] @ w[pre + "right.o"].T
    return m["left_scale"] * left + m["right_scale"] * right


def mixer(kind, h, m, w, pre, eps):
    if kind == "latent_attention":
        return latent_attention(h, m, w, pre, eps)
    if kind == "attention":
        return pooled_attention(h, m, w, pre)
    if kind == "parallel":
        return parallel_mixer(h, m, w, pre, eps)
    raise ValueError(kind)


def dense_ff(h, w, pre):
    return xielu(h @ w[pre + "up"].T, w[pre + "act"]) @ w[pre + "down"].T


# ---------------------------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------------------------
def layer_runs(cfg):
    """[(layer, pass number or None)]: the pass number stands at the first layer of every pass of the loop."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None) for i in range(a)]
    for t in range(times):
        runs += [(i, t if i == a else None) for i in range(a, b)]
    return runs + [(i, None) for i in range(b, n)]


def layer(x, i, cfg, w):
    L, eps, pre = cfg["layers"][i], cfg["norm"]["eps"], f"l{i}."
    a = mixer(L["type"], layer_norm(x, w[pre + "norm1"], eps), L["mixer"], w, pre + "mix.", eps)
    x = x + layer_norm(a, w[pre + "norm1b"], eps)
    if L.get("mlp") is not None:
        f = dense_ff(layer_norm(x, w[pre + "norm2"], eps), w, pre + "mlp.")
        x = x + layer_norm(f, w[pre + "norm2b"], eps)
    return x


def forward(cfg, w, ids, return_layers: bool = False):
    """Logits [n, vocab] for one sequence of token ids (and, if asked, the stream after every layer run)."""
    dtype = w["embed"].dtype
    x0 = w["embed"][torch.as_tensor(ids, dtype=torch.long)] * torch.tensor(cfg["embedding"]["scale"], dtype=dtype)
    x = x0
    after = []
    for i, t in layer_runs(cfg):
        if t is not None:
            if t > 0:
                x = x + x0
            x = x + w["loop.step"][t]
        x = layer(x, i, cfg, w)
        after.append(x)
    logits = layer_norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["head"].T
    return (logits, torch.stack(after)) if return_layers else logits


# ---------------------------------------------------------------------------------------------------------
# random weights for a configuration
# ---------------------------------------------------------------------------------------------------------
def tensor_shapes(cfg):
    W, V = cfg["width"], cfg["vocab"]
    s = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    if cfg.get("loop"):
        s["loop.step"] = (cfg["loop"]["times"], W)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        s[p + "norm1"] = s[p + "norm1b"] = (W,)
        if L["type"] == "parallel":
            l, r = m["left"], m["right"]
            s[p + "mix.left.q"] = (l["heads"] * l["dim"], W)
            s[p + "mix.left.k"] = (l["kv_heads"] * l["dim"], W)
            s[p + "mix.left.q.norm"] = (l["heads"] * l["dim"],)
            s[p + "mix.left.k.norm"] = (l["kv_heads"] * l["dim"],)
            s[p + "mix.left.g"] = (l["heads"] * l["vdim"], W)
            s[p + "mix.left.o"] = (W, l["heads"] * l["vdim"])
            for n in ("z", "x", "g"):
                s[p + "mix.right." + n] = (r["width"], W)
            s[p + "mix.right.z.b"] = s[p + "mix.right.x.b"] = (r["width"],)
            s[p + "mix.right.o"] = (W, r["width"])
        elif L["type"] == "latent_attention":
            H = m["heads"]
            s[p + "mix.dq"] = (m["q_rank"], W)
            s[p + "mix.dq.norm"] = (m["q_rank"],)
            s[p + "mix.uq"] = (H * (m["dim"] + m["rot_dim"]), m["q_rank"])
            s[p + "mix.dkv"] = (m["kv_rank"] + m["rot_dim"], W)
            s[p + "mix.dkv.norm"] = (m["kv_rank"],)
            s[p + "mix.uk"] = (H * m["dim"], m["kv_rank"])
            s[p + "mix.uv"] = (H * m["vdim"], m["kv_rank"])
            s[p + "mix.o"] = (W, H * m["vdim"])
        else:
            s[p + "mix.q"] = (m["heads"] * m["dim"], W)
            s[p + "mix.k"] = (m["kv_heads"] * m["dim"], W)
            s[p + "mix.o"] = (W, m["heads"] * m["vdim"])
        if L.get("mlp") is not None:
            s[p + "norm2"] = s[p + "norm2b"] = (W,)
            s[p + "mlp.up"] = (L["mlp"]["ff"], W)
            s[p + "mlp.down"] = (W, L["mlp"]["ff"])
            s[p + "mlp.act"] = (2,)
    return s


def random_weights(cfg, seed=0):
    """float32; matrices N(0, 1 / fan-in), norm weights around 1, biases and the pass vectors small."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        t = torch.randn(*shape, generator=g)
        if name.split(".")[-1].startswith("norm"):
            t = 1.0 + 0.1 * t
        elif name.endswith(".b"):
            t = 0.5 * t
        elif name == "loop.step":
            t = 0.3 * t
        elif name.endswith("mlp.act"):
            t = 0.5 * t
        elif name == "embed":
            t = t / math.sqrt(shape[1])
        else:
            t = t / math.sqrt(shape[-1])
        w[name] = t
    return w
