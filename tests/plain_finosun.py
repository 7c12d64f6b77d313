"""The Finosun decoder restated plainly: one slow function per mechanism, whole sequences at once, any float
dtype (the tests run it in 64-bit on the weights as given).  It shares no code with the engine.

Notation: n tokens, positions 0 .. n-1; x [n, width]; a linear map is `x @ W.T` with W [out, in].
"""

from __future__ import annotations

import math

import torch

# constants the design fixes
ACT_SLOPE = 1.702  # of the experts' gate: g * sigmoid(1.702 g)


# ---------------------------------------------------------------------------------------------------------
# norms, rotation
# ---------------------------------------------------------------------------------------------------------
def rms_norm(x, w, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def _angles(positions, dims, base, dtype):
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims).to(dtype)
    a = positions.to(dtype)[:, None] * f[None, :]
    return torch.cos(a), torch.sin(a)


def rotate_neighbours(v, positions, dims, base):
    """v [..., n, d]: (2i, 2i + 1), i < dims / 2, turn by position * base^(-2i / dims); the rest stays."""
    c, s = _angles(positions, dims, base, v.dtype)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out = v.clone()
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def rotate_halves(v, positions, dims, base):
    """v [..., n, d]: (i, i + dims / 2), i < dims / 2, turn by position * base^(-2i / dims); the rest stays."""
    c, s = _angles(positions, dims, base, v.dtype)
    h = dims // 2
    a, b = v[..., :h], v[..., h:dims]
    out = v.clone()
    out[..., :h] = a * c - b * s
    out[..., h:dims] = b * c + a * s
    return out


# ---------------------------------------------------------------------------------------------------------
# the softmax core (a loop over query positions: slow and plain)
# ---------------------------------------------------------------------------------------------------------
def masked_attention(q, k, v, factors, size):
    """q [H, n, d], k [G, n, d], v [G, n, dv], factors [H] (what multiplies a head's scores) -> [n, H * dv].
    Query i sees j with 0 <= i - j < size (None: every j <= i)."""
    H, n, _ = q.shape
    G, dv = k.shape[0], v.shape[-1]
    rep = H // G
    out = torch.zeros(n, H, dv, dtype=q.dtype)
    for i in range(n):
        lo = 0 if size is None else max(0, i - size + 1)
        for h in range(H):
            g = h // rep
            s = (k[g, lo:i + 1] @ q[h, i]) * factors[h]
            p = torch.softmax(s, 0)
            out[i, h] = p @ v[g, lo:i + 1]
    return out.reshape(n, H * dv)


# ---------------------------------------------------------------------------------------------------------
# mixers
# ---------------------------------------------------------------------------------------------------------
def grouped_attention(h, m, w, pre, eps):
    """Grouped heads; q and k normed over the whole projection (a weight per channel) before the rotation of
    neighbours; every head's value divided by its root mean square; a factor per head on the scores; a window."""
    n = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(n)
    q = rms_norm(h @ w[pre + "q"].T, w[pre + "q.norm"], eps).reshape(n, H, d).transpose(0, 1)
    k = rms_norm(h @ w[pre + "k"].T, w[pre + "k.norm"], eps).reshape(n, G, d).transpose(0, 1)
    v = rms_norm((h @ w[pre + "v"].T).reshape(n, G, dv), None, eps).transpose(0, 1)
    rot = m.get("rot")
    if rot:
        q = rotate_neighbours(q, pos, rot["dims"], rot["base"])
        k = rotate_neighbours(k, pos, rot["dims"], rot["base"])
    factors = w[pre + "temp"].to(h.dtype) * m["scale"]
    size = m["mask"]["size"] if m.get("mask") else None
    return masked_attention(q, k, v, factors, size) @ w[pre + "o"].T


def latent_attention(h, m, w, pre, eps):
    """Keys and values from one normed latent per token plus one rotated key part that all heads share; queries
    projected directly; causal; the heads' outputs pass a sigmoid gate read from the mixer's input."""
    n = h.shape[0]
    H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(n)
    q = (h @ w[pre + "q"].T).reshape(n, H, d + r).transpose(0, 1)
    down = h @ w[pre + "dkv"].T
    c = rms_norm(down[:, :R], w[pre + "dkv.norm"], eps)
    k_plain = (c @ w[pre + "uk"].T).reshape(n, H, d).transpose(0, 1)
    v = (c @ w[pre + "uv"].T).reshape(n, H, dv).transpose(0, 1)
    q_rot, k_rot = q[..., d:], down[None, :, R:]
    if r:
        q_rot = rotate_halves(q_rot, pos, r, m["rot"]["base"])
        k_rot = rotate_halves(k_rot, pos, r, m["rot"]["base"])
    qq = torch.cat([q[..., :d], q_rot], -1)
    kk = torch.cat([k_plain, k_rot.expand(H, n, r)], -1)
    size = m["mask"]["size"] if m.get("mask") else None
    a = masked_attention(qq, kk, v, torch.full((H,), float(m["scale"]), dtype=h.dtype), size)
    a = a * torch.sigmoid(h @ w[pre + "g"].T)
    return a @ w[pre + "o"].T


def mixer(kind, h, m, w, pre, eps):
    if kind == "attention":
        return grouped_attention(h, m, w, pre, eps)
    if kind == "latent_attention":
        return latent_attention(h, m, w, pre, eps)
    raise ValueError(kind)


# ---------------------------------------------------------------------------------------------------------
# feed-forward
# ---------------------------------------------------------------------------------------------------------
def expert(h, w, pre, limit):
    g = torch.clamp(h @ w[pre + "gate"].T, max=limit)
    u = torch.clamp(h @ w[pre + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(ACT_SLOPE * g) * (u + 1)) @ w[pre + "down"].T


def route(h, w, pre, top):
    """(chosen [n, top], their weights [n, top]): softmax over all router outputs; the choice adds a correction
    per output, the weight does not, and is not renormalized.  Ties go to the lower index."""
    s = torch.softmax(h @ w[pre + "router"].T, -1)
    chosen = torch.topk(s + w[pre + "correction"].to(s.dtype), top, dim=-1, sorted=True).indices
    return chosen, torch.gather(s, 1, chosen)


def routed_ff(h, f, w, pre):
    E, ident, top = f["router"]["experts"], f["router"].get("identity", 0), f["router"]["top"]
    chosen, weight = route(h, w, pre, top)
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(chosen[t, j])
            if e >= E:  # one of the last `ident` outputs: the input passes
                assert e < E + ident
                y[t] += weight[t, j] * h[t]
            else:
                y[t] += weight[t, j] * expert(h[t:t + 1], w, f"{pre}e{e}.", f["expert"]["limit"])[0]
    if f.get("shared"):
        gate = torch.sigmoid(h @ w[pre + "shared.sg"].T)  # [n, 1]
        y = y + gate * expert(h, w, pre + "shared.", f["shared"]["limit"])
    return y


# ---------------------------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------------------------
def layer_runs(cfg):
    """[(layer, starts a pass)] in the order the layers run."""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return [(i, False) for i in range(n)]
    a, b, times = lp["start"], lp["stop"], lp["times"]
    runs = [(i, False) for i in range(a)]
    for _ in range(times):
        runs += [(i, i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b, n)]


def layer(x, i, cfg, w):
    L, eps, pre = cfg["layers"][i], cfg["norm"]["eps"], f"l{i}."
    a = mixer(L["type"], rms_norm(x, w[pre + "norm1"], eps), L["mixer"], w, pre + "mix.", eps)
    x = x + w[pre + "ls1"] * a
    if L.get("mlp") is not None:
        f = routed_ff(rms_norm(x, w[pre + "norm2"], eps), L["mlp"], w, pre + "mlp.")
        x = x + w[pre + "ls2"] * f
    return x


def forward(cfg, w, ids, return_layers: bool = False):
    """Logits [n, vocab] of one sequence (and the stream after every layer run, if asked)."""
    x0 = w["embed"][torch.as_tensor(ids, dtype=torch.long)]
    x, seen = x0, []
    for i, starts in layer_runs(cfg):
        if starts:
            x = torch.cat([x, x0], -1) @ w["loop.in"].T
        x = layer(x, i, cfg, w)
        seen.append(x)
    logits = rms_norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["embed"].T
    return (logits, torch.stack(seen)) if return_layers else logits


# ---------------------------------------------------------------------------------------------------------
# shapes and random weights
# ---------------------------------------------------------------------------------------------------------
def tensor_shapes(cfg):
    """{name: (shape, kind)}; kind: "matrix", "norm" (near 1), "scale" (a positive factor), "small"."""
    W, out = cfg["width"], {}
    out["embed"] = ((cfg["vocab"], W), "matrix")
    if cfg.get("loop"):
        out["loop.in"] = ((W, 2 * W), "matrix")
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = ((W,), "norm")
        out[p + "ls1"] = ((W,), "scale")
        if L["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out[p + "mix.q"] = ((H * d, W), "matrix")
            out[p + "mix.k"] = ((G * d, W), "matrix")
            out[p + "mix.v"] = ((G * dv, W), "matrix")
            out[p + "mix.q.norm"] = ((H * d,), "norm")
            out[p + "mix.k.norm"] = ((G * d,), "norm")
            out[p + "mix.temp"] = ((H,), "scale")
            out[p + "mix.o"] = ((W, H * dv), "matrix")
        else:
            H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            out[p + "mix.q"] = ((H * (d + r), W), "matrix")
            out[p + "mix.dkv"] = ((R + r, W), "matrix")
            out[p + "mix.dkv.norm"] = ((R,), "norm")
            out[p + "mix.uk"] = ((H * d, R), "matrix")
            out[p + "mix.uv"] = ((H * dv, R), "matrix")
            out[p + "mix.g"] = ((H * dv, W), "matrix")
            out[p + "mix.o"] = ((W, H * dv), "matrix")
        f = L.get("mlp")
        if f is not None:
            out[p + "norm2"] = ((W,), "norm")
            out[p + "ls2"] = ((W,), "scale")
            E, ident = f["router"]["experts"], f["router"].get("identity", 0)
            for e in range(E):
                out[f"{p}mlp.e{e}.gate"] = ((f["expert"]["ff"], W), "matrix")
                out[f"{p}mlp.e{e}.up"] = ((f["expert"]["ff"], W), "matrix")
                out[f"{p}mlp.e{e}.down"] = ((W, f["expert"]["ff"]), "matrix")
            out[p + "mlp.router"] = ((E + ident, W), "router")
            out[p + "mlp.correction"] = ((E + ident,), "small")
            if f.get("shared"):
                out[p + "mlp.shared.gate"] = ((f["shared"]["ff"], W), "matrix")
                out[p + "mlp.shared.up"] = ((f["shared"]["ff"], W), "matrix")
                out[p + "mlp.shared.down"] = ((W, f["shared"]["ff"]), "matrix")
                out[p + "mlp.shared.sg"] = ((1, W), "matrix")
    out["final.norm"] = ((W,), "norm")
    return out


def random_weights(cfg, seed=0):
    """float32 weights, each rounded to bfloat16 values so that every engine dtype holds the same numbers."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, (shape, kind) in tensor_shapes(cfg).items():
        if kind == "matrix":
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        elif kind == "router":
            t = torch.randn(shape, generator=g) * (2.0 / math.sqrt(shape[-1]))
        elif kind == "norm":
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif kind == "scale":
            t = 0.5 + torch.rand(shape, generator=g)
        else:
            t = 0.05 * torch.randn(shape, generator=g)
        w[name] = t.to(torch.bfloat16).float()
    return w
